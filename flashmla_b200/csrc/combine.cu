// Split-KV combine: merges the partial results of requests that the tile scheduler split over
// several partitions.
//
// For one (request, query token, head) with n > 1 parts, part i carries a normalised fp32 output
// o_i[512] and a base-2 log-sum-exp L_i (-inf for a part that saw no valid token):
//   L   = log2(sum_i 2^L_i)            lse = L * ln2 (natural log; +inf when every part is empty)
//   L'  = L + log2(1 + 2^(sink*log2e - L))   when an attention sink is given (out is rescaled, lse is not)
//   out = sum_i 2^(L_i - L') * o_i     -> bf16
// Requests with exactly one part were written in final form by the attention kernel and are skipped.
// Same arithmetic as the reference's combine step (csrc/smxx/decode/combine/combine.cu:71-161).
//
// One warp per head, 8 heads per block; each lane owns 16 of the 512 output columns as 4 float4.
// HBM-bound: reads n*512*4 B and writes 512*2 B per (query, head).
#include <math_constants.h>

#include "common.cuh"

namespace fmla {

constexpr int COMBINE_HEADS_PER_BLOCK = 8;

__global__ void __launch_bounds__(COMBINE_HEADS_PER_BLOCK * 32)
combine_kernel(int s_q, int h_q, const int* __restrict__ num_splits, const float* __restrict__ o_accum,
               const float* __restrict__ lse_accum, const float* __restrict__ attn_sink,
               __nv_bfloat16* __restrict__ out, int64_t o_stride_b, int64_t o_stride_s, int64_t o_stride_h,
               float* __restrict__ lse, int64_t lse_stride_b, int64_t lse_stride_s) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int batch = blockIdx.x / s_q, sq = blockIdx.x % s_q;
  const int head = blockIdx.y * COMBINE_HEADS_PER_BLOCK + warp;
  // The kernel may have been launched while the attention kernel was still running (programmatic dependent
  // launch): its partial results are complete and visible only after this wait.  Every thread runs it, also
  // those that have nothing to merge: a grid whose blocks all left before the wait would complete ahead of the
  // attention kernel, and the next kernel in the stream - ordered behind this grid only - could then read
  // `out` / `lse` of unsplit requests while the attention kernel was still writing them.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (head >= h_q) return;
  const int first = num_splits[batch], n = num_splits[batch + 1] - first;
  if (n <= 1) return;

  const int64_t part_stride_lse = (int64_t)s_q * h_q;
  const int64_t part_stride_o = part_stride_lse * D_V;
  const float* lse_p = lse_accum + (int64_t)first * part_stride_lse + (int64_t)sq * h_q + head;
  const float* o_p = o_accum + (int64_t)first * part_stride_o + ((int64_t)sq * h_q + head) * D_V + lane * 4;

  // pass 1: global log-sum-exp (base 2) over the parts
  float mx = -CUDART_INF_F;
  for (int i = lane; i < n; i += 32) mx = fmaxf(mx, lse_p[i * part_stride_lse]);
#pragma unroll
  for (int off = 16; off; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  const float mx_safe = mx == -CUDART_INF_F ? 0.f : mx;
  float sum = 0.f;
  for (int i = lane; i < n; i += 32) sum += exp2f(lse_p[i * part_stride_lse] - mx_safe);
#pragma unroll
  for (int off = 16; off; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  float L = sum == 0.f ? CUDART_INF_F : log2f(sum) + mx_safe;
  if (lane == 0) lse[batch * lse_stride_b + sq * lse_stride_s + head] = L == CUDART_INF_F ? CUDART_INF_F : L * LN2;
  if (attn_sink != nullptr) {
    const float sink = attn_sink[head];
    if (L != CUDART_INF_F) L += log2f(1.f + exp2f(sink * LOG2E - L));   // sink=+inf -> L=+inf -> all weights 0
    else L = sink == -CUDART_INF_F ? CUDART_INF_F : sink * LOG2E;
  }

  // pass 2: weighted sum of the parts
  float4 acc[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) acc[c] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int i = 0; i < n; ++i) {
    const float w = exp2f(lse_p[i * part_stride_lse] - L);   // 2^(-inf) = 0 for empty parts
    const float* src = o_p + i * part_stride_o;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const float4 v = *reinterpret_cast<const float4*>(src + c * 128);
      acc[c].x += w * v.x; acc[c].y += w * v.y; acc[c].z += w * v.z; acc[c].w += w * v.w;
    }
  }
  __nv_bfloat16* dst = out + batch * o_stride_b + sq * o_stride_s + head * o_stride_h + lane * 4;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint2 packed = make_uint2(pack_bf16x2(acc[c].x, acc[c].y), pack_bf16x2(acc[c].z, acc[c].w));
    *reinterpret_cast<uint2*>(dst + c * 128) = packed;
  }
}

int launch_combine(const FmlaDecodeArgs& a, cudaStream_t stream) {
  dim3 grid(a.b * a.s_q, (a.h_q + COMBINE_HEADS_PER_BLOCK - 1) / COMBINE_HEADS_PER_BLOCK);
  // Launched as a programmatic dependent of the attention kernel, which precedes it in the stream: its blocks may
  // become resident as that kernel's blocks retire, and wait inside for its completion.  (With a timing event
  // between the two kernels the launch is an ordinary one.)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(COMBINE_HEADS_PER_BLOCK * 32);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = a.attn_done_event == nullptr ? 1 : 0;
  FMLA_CUDA(cudaLaunchKernelEx(&cfg, combine_kernel, a.s_q, a.h_q, a.num_splits, (const float*)a.o_accum, (const float*)a.lse_accum,
                               a.attn_sink, reinterpret_cast<__nv_bfloat16*>(a.out), a.o_stride_b, a.o_stride_s, a.o_stride_h,
                               a.lse, a.lse_stride_b, a.lse_stride_s));
  return FMLA_OK;
}

}  // namespace fmla
