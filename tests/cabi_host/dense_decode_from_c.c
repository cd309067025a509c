/* A host written in plain C drives the dense decode through the C ABI alone (no Python, no torch):
 * plan -> tile scheduler (lengths = cache_seqlens) -> fmla_dense_decode, on a bf16 cache whose rows are all the same
 * vector, where the answer is known in closed form: out = that vector's first 512 dims, and with `causal`
 * lse[row j of s_q] = sm_scale * (q . k) + ln(len - (s_q - 1 - j)).  The block table is a permutation with one entry
 * that lies outside the cache (its 64 tokens count as invalid slots).  Prints "OK" and returns 0 on success.
 * Build: see tests/test_gpu_cabi_c_host.py. */
#include <cuda_runtime_api.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "flashmla_b200.h"

#define CHECK_CUDA(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { fprintf(stderr, "CUDA: %s (%s:%d)\n", cudaGetErrorString(e_), __FILE__, __LINE__); return 2; } } while (0)
#define CHECK_FMLA(x) do { int rc_ = (x); if (rc_ != FMLA_OK) { fprintf(stderr, "fmla error %d: %s (%s:%d)\n", rc_, fmla_last_error(), __FILE__, __LINE__); return 3; } } while (0)

static uint16_t bf16_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16); }
static float bf16_value(uint16_t b) { uint32_t u = (uint32_t)b << 16; float f; memcpy(&f, &u, 4); return f; }

int main(void) {
  enum { b = 3, s_q = 2, h_q = 128, page = 64, num_blocks = 40, max_blocks = 12 };
  const int lens[b] = {700, 64, 333};           /* request 0 loses the 64 tokens of its hole: 636 remain */
  const float sm_scale = 0.05f, kval = 0.25f;
  const size_t rows = (size_t)num_blocks * page;

  uint16_t* h_kv = (uint16_t*)malloc(rows * FMLA_D_QK * 2);
  for (size_t i = 0; i < rows * FMLA_D_QK; ++i) h_kv[i] = bf16_bits(kval);
  const size_t nq = (size_t)b * s_q * h_q * FMLA_D_QK;
  uint16_t* h_q_bits = (uint16_t*)malloc(nq * 2);
  for (size_t i = 0; i < nq; ++i) {
    const int head = (int)((i / FMLA_D_QK) % h_q);
    h_q_bits[i] = bf16_bits(0.03125f * (float)(1 + head % 5));
  }
  int32_t h_bt[b * max_blocks];
  for (int i = 0; i < b; ++i)
    for (int j = 0; j < max_blocks; ++j) h_bt[i * max_blocks + j] = (i * max_blocks + j * 7) % num_blocks;
  h_bt[0 * max_blocks + 3] = num_blocks + 9;    /* tokens 192..255 of request 0: no such block */

  int parts = 0, overhead = 0, block = 0;
  CHECK_FMLA(fmla_decode_plan(0, h_q, s_q, FMLA_KERNEL_TC, &parts, &overhead, &block));

  void *d_kv, *d_q, *d_bt, *d_len, *d_out, *d_lse, *d_meta, *d_splits, *d_oacc, *d_lacc, *d_status;
  CHECK_CUDA(cudaMalloc(&d_kv, rows * FMLA_D_QK * 2));
  CHECK_CUDA(cudaMalloc(&d_q, nq * 2));
  CHECK_CUDA(cudaMalloc(&d_bt, sizeof h_bt));
  CHECK_CUDA(cudaMalloc(&d_len, sizeof lens));
  CHECK_CUDA(cudaMalloc(&d_out, (size_t)b * s_q * h_q * FMLA_D_V * 2));
  CHECK_CUDA(cudaMalloc(&d_lse, (size_t)b * s_q * h_q * 4));
  CHECK_CUDA(cudaMalloc(&d_meta, (size_t)parts * 32));
  CHECK_CUDA(cudaMalloc(&d_splits, (size_t)(b + 1) * 4));
  CHECK_CUDA(cudaMalloc(&d_oacc, (size_t)(b + parts) * s_q * h_q * FMLA_D_V * 4));
  CHECK_CUDA(cudaMalloc(&d_lacc, (size_t)(b + parts) * s_q * h_q * 4));
  CHECK_CUDA(cudaMalloc(&d_status, 4));
  CHECK_CUDA(cudaMemset(d_status, 0, 4));
  CHECK_CUDA(cudaMemcpy(d_kv, h_kv, rows * FMLA_D_QK * 2, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(d_q, h_q_bits, nq * 2, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(d_bt, h_bt, sizeof h_bt, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(d_len, lens, sizeof lens, cudaMemcpyHostToDevice));

  FmlaSchedArgs sa;
  memset(&sa, 0, sizeof sa);
  sa.device = 0; sa.b = b; sa.topk = max_blocks * page; sa.block_topk = block; sa.fixed_overhead_blocks = overhead; sa.num_sm_parts = parts;
  sa.topk_length = (const int32_t*)d_len;
  sa.sched_meta = (int32_t*)d_meta; sa.num_splits = (int32_t*)d_splits;
  CHECK_FMLA(fmla_sched_meta(&sa, NULL));

  FmlaDenseDecodeArgs da;
  memset(&da, 0, sizeof da);
  da.device = 0; da.b = b; da.s_q = s_q; da.h_q = h_q; da.causal = 1; da.sm_scale = sm_scale;
  da.q = d_q; da.q_stride_b = (int64_t)s_q * h_q * FMLA_D_QK; da.q_stride_s = (int64_t)h_q * FMLA_D_QK; da.q_stride_h = FMLA_D_QK;
  da.kv = d_kv; da.num_blocks = num_blocks; da.page_block_size = page; da.kv_stride_row = FMLA_D_QK;
  da.block_table = (const int32_t*)d_bt; da.block_table_stride = max_blocks; da.max_blocks_per_seq = max_blocks;
  da.cache_seqlens = (const int32_t*)d_len;
  da.out = d_out; da.o_stride_b = (int64_t)s_q * h_q * FMLA_D_V; da.o_stride_s = (int64_t)h_q * FMLA_D_V; da.o_stride_h = FMLA_D_V;
  da.lse = (float*)d_lse; da.lse_stride_b = (int64_t)s_q * h_q; da.lse_stride_s = h_q;
  da.sched_meta = (const int32_t*)d_meta; da.num_splits = (const int32_t*)d_splits; da.num_sm_parts = parts;
  da.o_accum = (float*)d_oacc; da.lse_accum = (float*)d_lacc; da.status = (int32_t*)d_status;
  CHECK_FMLA(fmla_dense_decode(&da, NULL));
  CHECK_CUDA(cudaDeviceSynchronize());

  uint16_t* h_out = (uint16_t*)malloc((size_t)b * s_q * h_q * FMLA_D_V * 2);
  float* h_lse = (float*)malloc((size_t)b * s_q * h_q * 4);
  int32_t status = -1;
  CHECK_CUDA(cudaMemcpy(h_out, d_out, (size_t)b * s_q * h_q * FMLA_D_V * 2, cudaMemcpyDeviceToHost));
  CHECK_CUDA(cudaMemcpy(h_lse, d_lse, (size_t)b * s_q * h_q * 4, cudaMemcpyDeviceToHost));
  CHECK_CUDA(cudaMemcpy(&status, d_status, 4, cudaMemcpyDeviceToHost));
  if (status != 0) { fprintf(stderr, "kernel status %d\n", status); return 4; }

  int bad = 0;
  for (int i = 0; i < b * s_q * h_q && bad < 5; ++i) {
    const int head = i % h_q, sq = (i / h_q) % s_q, req = i / (h_q * s_q);
    int seen = lens[req] - (s_q - 1 - sq);
    if (req == 0) seen -= 64;                    /* the hole lies below both rows' limits */
    const float qv = bf16_value(bf16_bits(0.03125f * (float)(1 + head % 5)));
    const float dot = qv * (float)FMLA_D_QK * kval;
    const float want_lse = sm_scale * dot + logf((float)seen);
    if (fabsf(h_lse[i] - want_lse) > 1e-3f * fmaxf(1.0f, fabsf(want_lse))) { fprintf(stderr, "lse[%d] = %f, want %f\n", i, h_lse[i], want_lse); ++bad; }
    for (int d = 0; d < FMLA_D_V; d += 37) {
      const float o = bf16_value(h_out[(size_t)i * FMLA_D_V + d]);
      if (fabsf(o - kval) > 2e-2f * kval) { fprintf(stderr, "out[%d][%d] = %f, want %f\n", i, d, o, kval); ++bad; break; }
    }
  }
  if (bad) return 5;
  printf("OK dense h_q=%d parts=%d version=%d\n", (int)h_q, parts, fmla_version());
  return 0;
}
