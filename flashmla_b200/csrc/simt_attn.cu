// Generic CUDA-core sparse MLA attention kernels: decode over the paged FP8/MXFP8 cache, prefill
// forward, and prefill backward.  They accept any number of query heads and serve the shapes the
// tensor-core kernels do not cover.
//
// Work decomposition: one thread block per (query token, group of 16 heads) [times the split-KV
// partition for decode].  Per tile of 32 indexed tokens the block
//   1. gathers the rows into shared memory (FP8 rows are dequantised on the way: fp8 -> fp32 * scale
//      -> bf16, exactly the reference's dequantisation, tests/quant.py:93-104),
//   2. computes the 16x32 logits in fp32 (base-2 domain: x = q.k * sm_scale * log2e),
//   3. runs the online softmax update (running max m, running sum l), and
//   4. accumulates P.V into fp32 registers (each thread owns 32 of a head's 512 output columns).
// Invalid slots (index -1 / outside the cache, or position >= topk_length) are never loaded: their
// row is zero-filled and their logit is -inf, so they contribute exact zeros.
//
// Numerics follow the reference's oracle (tests/ref.py:19-103): lse is the natural log-sum-exp of the
// valid logits, a query row without valid slot yields out = 0 and lse = +inf, and attn_sink rescales
// out by 1/(1+exp(sink-lse)) without touching lse.
#include <math_constants.h>

#include <type_traits>

#include "common.cuh"

namespace fmla {
namespace simt {

constexpr int HG = 16;        // heads per block
constexpr int TILE = 32;      // tokens per tile
constexpr int THREADS = 256;
constexpr int KV_W = 292;     // 32-bit words per KV row in smem (288 + pad; 292 % 32 == 4 keeps 16-B loads conflict free)
constexpr int Q_W = 292;      // words per Q row
constexpr int DO_W = 260;     // words per dO row (256 + pad)

// ---------------------------------------------------------------------------------------------
// Row sources
// ---------------------------------------------------------------------------------------------
struct PagedFp8Rows {
  const uint8_t* base;
  int64_t block_stride;   // bytes
  int page;
  int64_t total_rows;
  int layout;
  __device__ __forceinline__ bool in_range(int idx) const { return idx >= 0 && idx < total_rows; }
  __device__ __forceinline__ const uint8_t* row(int idx) const {
    const int blk = idx / page, off = idx - blk * page;
    return base + blk * block_stride + (int64_t)off * ROW_BYTES;
  }
};

struct Bf16Rows {
  const __nv_bfloat16* base;
  int64_t stride;         // elements
  int64_t total_rows;
  int chunks;             // 16-byte chunks per row: 72 (d_qk = 576) or 64 (d_qk = 512; the row is zero-padded to 576 in shared memory)
  __device__ __forceinline__ bool in_range(int idx) const { return idx >= 0 && idx < total_rows; }
  __device__ __forceinline__ const __nv_bfloat16* row(int idx) const { return base + idx * stride; }
};

// MODEL1 cache blocks (tests/quant.py:55-75 of the reference): [page x (448 e4m3 | 64 bf16)] [page x (7 e8m0 | pad)].
struct PagedModel1Rows {
  const uint8_t* base;
  int64_t block_stride;   // bytes
  int page;
  int64_t total_rows;
  __device__ __forceinline__ bool in_range(int idx) const { return idx >= 0 && idx < total_rows; }
};

template <class Rows> __device__ __forceinline__ Rows make_paged_rows(const void* base, int64_t block_stride, int64_t page, int64_t blocks, int layout);
template <> __device__ __forceinline__ PagedFp8Rows make_paged_rows<PagedFp8Rows>(const void* base, int64_t block_stride, int64_t page, int64_t blocks, int layout) {
  return PagedFp8Rows{reinterpret_cast<const uint8_t*>(base), block_stride, (int)page, blocks * page, layout};
}
template <> __device__ __forceinline__ PagedModel1Rows make_paged_rows<PagedModel1Rows>(const void* base, int64_t block_stride, int64_t page, int64_t blocks, int) {
  return PagedModel1Rows{reinterpret_cast<const uint8_t*>(base), block_stride, (int)page, blocks * page};
}

// Dequantises 16 fp8 values (one uint4) with one scale into 8 bf16x2 words.
__device__ __forceinline__ void dequant16(const uint4& raw, float scale, uint32_t* dst /*8 words, 16-B aligned*/) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 a = e4m3x2_to_float2((uint16_t)(w[i] & 0xffffu));
    const float2 b = e4m3x2_to_float2((uint16_t)(w[i] >> 16));
    o[2 * i] = pack_bf16x2(a.x * scale, a.y * scale);
    o[2 * i + 1] = pack_bf16x2(b.x * scale, b.y * scale);
  }
  *reinterpret_cast<uint4*>(dst) = make_uint4(o[0], o[1], o[2], o[3]);
  *reinterpret_cast<uint4*>(dst + 4) = make_uint4(o[4], o[5], o[6], o[7]);
}

// Loads one row into smem (as 288 bf16x2 words), cooperatively by `nsub` threads (sub = 0..nsub-1).
__device__ __forceinline__ void load_row(const PagedFp8Rows& src, int idx, bool valid, uint32_t* dst, int sub, int nsub) {
  if (!valid) {
    for (int c = sub; c < 72; c += nsub) *reinterpret_cast<uint4*>(dst + 4 * c) = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint8_t* r = src.row(idx);
  const uint4 sc = ldg_nc_16(r + SCALE_OFF);
  for (int c = sub; c < 32; c += nsub) {       // 32 chunks of 16 fp8
    const uint4 raw = ldg_nc_16(r + 16 * c);
    float scale;
    if (src.layout == FMLA_LAYOUT_V32) {
      const uint32_t sw[4] = {sc.x, sc.y, sc.z, sc.w};
      scale = __uint_as_float(sw[c >> 3]);
    } else {
      const uint32_t sw[4] = {sc.x, sc.y, sc.z, sc.w};
      const int k = c >> 1;                     // one e8m0 byte per 32 elements
      scale = e8m0_to_float((sw[k >> 2] >> (8 * (k & 3))) & 0xffu);
    }
    dequant16(raw, scale, dst + 8 * c);
  }
  for (int c = sub; c < 8; c += nsub)          // 64 bf16 RoPE values, copied verbatim
    *reinterpret_cast<uint4*>(dst + 256 + 4 * c) = ldg_nc_16(r + ROPE_OFF + 16 * c);
}

__device__ __forceinline__ void load_row(const Bf16Rows& src, int idx, bool valid, uint32_t* dst, int sub, int nsub) {
  if (!valid) {
    for (int c = sub; c < 72; c += nsub) *reinterpret_cast<uint4*>(dst + 4 * c) = make_uint4(0, 0, 0, 0);
    return;
  }
  const __nv_bfloat16* r = src.row(idx);
  for (int c = sub; c < 72; c += nsub)
    *reinterpret_cast<uint4*>(dst + 4 * c) = c < src.chunks ? ldg_nc_16(r + 8 * c) : make_uint4(0, 0, 0, 0);
}

// A MODEL1 row as 512 values (448 dequantised exactly as tests/quant.py:106-118 does: e4m3 times a power-of-two
// e8m0 scale in bf16, which is exact; then the 64 RoPE values), zero-padded to the 576-wide shared-memory row.
__device__ __forceinline__ void load_row(const PagedModel1Rows& src, int idx, bool valid, uint32_t* dst, int sub, int nsub) {
  if (!valid) {
    for (int c = sub; c < 72; c += nsub) *reinterpret_cast<uint4*>(dst + 4 * c) = make_uint4(0, 0, 0, 0);
    return;
  }
  const int blk = idx / src.page, off = idx - blk * src.page;
  const uint8_t* block = src.base + blk * src.block_stride;
  const uint8_t* r = block + (int64_t)off * M1_DATA_BYTES;
  const uint2 sc = *reinterpret_cast<const uint2*>(block + (int64_t)src.page * M1_DATA_BYTES + 8 * off);
  for (int c = sub; c < 28; c += nsub) {       // 28 chunks of 16 fp8; one scale byte per 64 values = 4 chunks
    const int k = c >> 2;
    const float scale = e8m0_to_float(((k < 4 ? sc.x : sc.y) >> (8 * (k & 3))) & 0xffu);
    dequant16(ldg_nc_16(r + 16 * c), scale, dst + 8 * c);
  }
  for (int c = sub; c < 8; c += nsub)          // 64 bf16 RoPE values = dims 448 .. 511
    *reinterpret_cast<uint4*>(dst + 224 + 4 * c) = ldg_nc_16(r + M1_D_NOPE + 16 * c);
  for (int c = sub; c < 8; c += nsub)          // padding up to 576
    *reinterpret_cast<uint4*>(dst + 256 + 4 * c) = make_uint4(0, 0, 0, 0);
}

__device__ __forceinline__ float dot_words(const uint4& a, const uint4& b, float acc) {
  const uint32_t x[4] = {a.x, a.y, a.z, a.w}, y[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc = fmaf(bf16_bits_to_float(x[i] & 0xffffu), bf16_bits_to_float(y[i] & 0xffffu), acc);
    acc = fmaf(__uint_as_float(x[i] & 0xffff0000u), __uint_as_float(y[i] & 0xffff0000u), acc);
  }
  return acc;
}

// ---------------------------------------------------------------------------------------------
// Forward core shared by decode and prefill
// ---------------------------------------------------------------------------------------------
struct FwdSmem {
  uint32_t q[HG * Q_W];
  uint32_t kv[TILE * KV_W];
  float p[HG * TILE];
  float m[HG], l[HG], alpha[HG];
  int valid[TILE];
};

// Loads the bf16 query rows of this head group (rows beyond h_q are zero).
// `chunks` = 16-byte chunks per query row (72, or 64 for d_qk = 512: the rest of the 576-wide row is zero).
__device__ __forceinline__ void load_q_group(uint32_t* q_s, const __nv_bfloat16* q, int64_t stride_h, int head0, int h_q, int chunks = 72) {
  for (int i = threadIdx.x; i < HG * 72; i += THREADS) {
    const int h = i / 72, c = i % 72;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (head0 + h < h_q && c < chunks) v = ldg_nc_16(q + (head0 + h) * stride_h + 8 * c);
    *reinterpret_cast<uint4*>(q_s + h * Q_W + 4 * c) = v;
  }
}

// Processes index slots [tok_lo, tok_hi) of one query.  acc[32]: thread (h = tid/16, g = tid%16) owns
// output elements 8g + 128i + (0..7), i = 0..3, of head h.  m/l live in smem.
template <class Rows>
__device__ __forceinline__ void attend(FwdSmem& s, const Rows& rows, const int* __restrict__ idx, int tok_lo, int tok_hi,
                                       int valid_limit, float scale_log2, float (&acc)[32]) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int t0 = tok_lo; t0 < tok_hi; t0 += TILE) {
    {  // gather: 8 threads per token
      const int j = tid >> 3, sub = tid & 7;
      const int pos = t0 + j;
      int id = -1;
      if (pos < tok_hi && pos < valid_limit) id = __ldg(idx + pos);
      const bool ok = rows.in_range(id);
      load_row(rows, id, ok, s.kv + j * KV_W, sub, 8);
      if (sub == 0) s.valid[j] = ok;
    }
    __syncthreads();
    {  // logits: lane -> head (lane&15), tokens 4*warp + (lane>>4) and +2
      const int h = lane & 15, j0 = 4 * warp + (lane >> 4), j1 = j0 + 2;
      const uint4* qp = reinterpret_cast<const uint4*>(s.q + h * Q_W);
      const uint4* k0 = reinterpret_cast<const uint4*>(s.kv + j0 * KV_W);
      const uint4* k1 = reinterpret_cast<const uint4*>(s.kv + j1 * KV_W);
      float a0 = 0.f, a1 = 0.f;
#pragma unroll 4
      for (int c = 0; c < 72; ++c) {
        const uint4 qv = qp[c];
        a0 = dot_words(qv, k0[c], a0);
        a1 = dot_words(qv, k1[c], a1);
      }
      s.p[h * TILE + j0] = s.valid[j0] ? a0 * scale_log2 : -CUDART_INF_F;
      s.p[h * TILE + j1] = s.valid[j1] ? a1 * scale_log2 : -CUDART_INF_F;
    }
    __syncthreads();
    {  // online softmax: warp handles heads 2*warp, 2*warp+1; lane <-> token
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int h = 2 * warp + hh;
        const float x = s.p[h * TILE + lane];
        float mx = x;
#pragma unroll
        for (int off = 16; off; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        const float m_old = s.m[h];
        const float m_new = fmaxf(m_old, mx);
        float p = 0.f, alpha = 1.f;
        if (m_new != -CUDART_INF_F) {
          alpha = exp2f(m_old - m_new);
          p = exp2f(x - m_new);
        }
        float sum = p;
#pragma unroll
        for (int off = 16; off; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        s.p[h * TILE + lane] = p;
        if (lane == 0) {
          s.m[h] = m_new;
          s.l[h] = s.l[h] * alpha + sum;
          s.alpha[h] = alpha;
        }
      }
    }
    __syncthreads();
    {  // P.V
      const int h = tid >> 4, g = tid & 15;
      const float alpha = s.alpha[h];
#pragma unroll
      for (int e = 0; e < 32; ++e) acc[e] *= alpha;
      for (int j = 0; j < TILE; ++j) {
        const float p = s.p[h * TILE + j];
        const uint32_t* vrow = s.kv + j * KV_W + 4 * g;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint4 v = *reinterpret_cast<const uint4*>(vrow + 64 * i);
          const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            acc[8 * i + 2 * k] = fmaf(p, bf16_bits_to_float(w[k] & 0xffffu), acc[8 * i + 2 * k]);
            acc[8 * i + 2 * k + 1] = fmaf(p, __uint_as_float(w[k] & 0xffff0000u), acc[8 * i + 2 * k + 1]);
          }
        }
      }
    }
    __syncthreads();
  }
}

__device__ __forceinline__ void reset_state(FwdSmem& s, float (&acc)[32]) {
  if (threadIdx.x < HG) {
    s.m[threadIdx.x] = -CUDART_INF_F;
    s.l[threadIdx.x] = 0.f;
    s.alpha[threadIdx.x] = 1.f;
  }
#pragma unroll
  for (int e = 0; e < 32; ++e) acc[e] = 0.f;
}

__device__ __forceinline__ void store_bf16_row(__nv_bfloat16* dst, const float (&acc)[32], float mul, int g) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 v;
    v.x = pack_bf16x2(acc[8 * i + 0] * mul, acc[8 * i + 1] * mul);
    v.y = pack_bf16x2(acc[8 * i + 2] * mul, acc[8 * i + 3] * mul);
    v.z = pack_bf16x2(acc[8 * i + 4] * mul, acc[8 * i + 5] * mul);
    v.w = pack_bf16x2(acc[8 * i + 6] * mul, acc[8 * i + 7] * mul);
    *reinterpret_cast<uint4*>(dst + 8 * g + 128 * i) = v;
  }
}

// 1/(l + 2^(sink*log2e - m)): the factor that normalises the accumulator and applies the sink.
__device__ __forceinline__ float final_scale(float m, float l, const float* attn_sink, int head) {
  if (l == 0.f) return 0.f;
  float denom = l;
  if (attn_sink != nullptr) denom += exp2f(attn_sink[head] * LOG2E - m);
  return 1.f / denom;     // sink = +inf -> denom = inf -> 0
}

// ---------------------------------------------------------------------------------------------
// Decode
// ---------------------------------------------------------------------------------------------
template <class Rows>
__global__ void __launch_bounds__(THREADS)
decode_kernel(const FmlaDecodeArgs a, int block_topk) {
  constexpr int q_chunks = std::is_same<Rows, PagedModel1Rows>::value ? 64 : 72;     // MODEL1: d_qk = 512
  extern __shared__ __align__(16) uint8_t smem_raw[];
  FwdSmem& s = *reinterpret_cast<FwdSmem*>(smem_raw);
  const int part = blockIdx.x, sq = blockIdx.y, head0 = blockIdx.z * HG;
  const SchedRecord rec = reinterpret_cast<const SchedRecord*>(a.sched_meta)[part];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the combine kernel may start launching; it waits for this grid itself
  if (rec.begin_req >= a.b) return;
  const Rows rows = make_paged_rows<Rows>(a.kv, a.kv_stride_block, a.page_block_size, a.num_blocks, a.layout);
  const float scale_log2 = a.sm_scale * LOG2E;
  const int tid = threadIdx.x, h = tid >> 4, g = tid & 15, head = head0 + h;
  float acc[32];

  for (int req = rec.begin_req; req <= rec.end_req; ++req) {
    const int blk_lo = req == rec.begin_req ? rec.begin_block : 0;
    const int blk_hi = req == rec.end_req ? rec.end_block : 0x3fffffff;
    const bool is_split = req == rec.begin_req ? rec.first_split : (req == rec.end_req ? rec.last_split : 0);
    const int limit_raw = a.topk_length ? __ldg(a.topk_length + req) : a.topk;
    const int limit = min(limit_raw, a.topk);
    // token list of the request: the main slots, then (with an extra cache) the extra slots from the next block boundary
    int main_end = a.topk, total = a.topk, extra_len = 0;
    if (a.extra_kv != nullptr) {
      const int s_main = limit_raw <= 0 ? 1 : limit_raw;
      main_end = (s_main + block_topk - 1) / block_topk * block_topk;
      extra_len = a.extra_topk_length ? __ldg(a.extra_topk_length + req) : a.extra_topk;
      extra_len = max(0, min(extra_len, a.extra_topk));
      total = main_end + extra_len;
    }
    const int tok_lo = blk_lo * block_topk;
    const int tok_hi = (int)min((int64_t)blk_hi * block_topk, (int64_t)total);

    __syncthreads();
    reset_state(s, acc);
    load_q_group(s.q, reinterpret_cast<const __nv_bfloat16*>(a.q) + req * a.q_stride_b + sq * a.q_stride_s,
                 a.q_stride_h, head0, a.h_q, q_chunks);
    __syncthreads();
    if (tok_lo < min(tok_hi, main_end))
      attend(s, rows, a.indices + req * a.idx_stride_b + sq * a.idx_stride_s, tok_lo, min(tok_hi, main_end), limit, scale_log2, acc);
    if (tok_hi > main_end) {
      const Rows extra_rows = make_paged_rows<Rows>(a.extra_kv, a.extra_kv_stride_block, a.extra_page_block_size, a.extra_num_blocks, a.layout);
      attend(s, extra_rows, a.extra_indices + req * a.extra_idx_stride_b + sq * a.extra_idx_stride_s, max(tok_lo, main_end) - main_end,
             tok_hi - main_end, extra_len, scale_log2, acc);
    }

    if (head < a.h_q) {
      const float m = s.m[h], l = s.l[h];
      if (is_split) {
        const int slot = __ldg(a.num_splits + req) + (req == rec.begin_req ? rec.begin_split : 0);
        const int64_t row = ((int64_t)slot * a.s_q + sq) * a.h_q + head;
        float* o = a.o_accum + row * D_V;
        const float inv = l == 0.f ? 0.f : 1.f / l;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          *reinterpret_cast<float4*>(o + 8 * g + 128 * i) =
              make_float4(acc[8 * i] * inv, acc[8 * i + 1] * inv, acc[8 * i + 2] * inv, acc[8 * i + 3] * inv);
          *reinterpret_cast<float4*>(o + 8 * g + 128 * i + 4) =
              make_float4(acc[8 * i + 4] * inv, acc[8 * i + 5] * inv, acc[8 * i + 6] * inv, acc[8 * i + 7] * inv);
        }
        if (g == 0) a.lse_accum[row] = l == 0.f ? -CUDART_INF_F : m + log2f(l);
      } else {
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(a.out) + req * a.o_stride_b + sq * a.o_stride_s + head * a.o_stride_h;
        store_bf16_row(o, acc, final_scale(m, l, a.attn_sink, head), g);
        if (g == 0) a.lse[req * a.lse_stride_b + sq * a.lse_stride_s + head] = l == 0.f ? CUDART_INF_F : (m + log2f(l)) * LN2;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Prefill forward
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(THREADS)
prefill_fwd_kernel(const FmlaPrefillArgs a) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  FwdSmem& s = *reinterpret_cast<FwdSmem*>(smem_raw);
  const int qi = blockIdx.x, head0 = blockIdx.y * HG;
  const int chunks = a.d_qk == M1_D_QK ? 64 : 72;
  const Bf16Rows rows{reinterpret_cast<const __nv_bfloat16*>(a.kv), a.kv_stride_s, a.s_kv, chunks};
  const int tid = threadIdx.x, h = tid >> 4, g = tid & 15, head = head0 + h;
  float acc[32];
  reset_state(s, acc);
  load_q_group(s.q, reinterpret_cast<const __nv_bfloat16*>(a.q) + qi * a.q_stride_s, a.q_stride_h, head0, a.h_q, chunks);
  __syncthreads();
  int limit = a.topk_length ? __ldg(a.topk_length + qi) : a.topk;
  limit = max(0, min(limit, a.topk));
  attend(s, rows, a.indices + qi * a.idx_stride_s, 0, limit, limit, a.sm_scale * LOG2E, acc);
  if (head < a.h_q) {
    const float m = s.m[h], l = s.l[h];
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(a.out) + ((int64_t)qi * a.h_q + head) * D_V;
    store_bf16_row(o, acc, final_scale(m, l, a.attn_sink, head), g);
    if (g == 0) {
      a.max_logits[(int64_t)qi * a.h_q + head] = l == 0.f ? -CUDART_INF_F : m * LN2;
      a.lse[(int64_t)qi * a.h_q + head] = l == 0.f ? CUDART_INF_F : (m + log2f(l)) * LN2;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Prefill backward
// ---------------------------------------------------------------------------------------------
// Base-2 log-sum-exp used to normalise P in the backward: the forward's lse merged with the sink.
__device__ __forceinline__ float lse_for_out_log2(float lse_nat, const float* attn_sink, int head) {
  if (lse_nat == CUDART_INF_F) return CUDART_INF_F;          // no valid token: P = 0 everywhere
  const float a = lse_nat * LOG2E;
  if (attn_sink == nullptr) return a;
  const float sk = attn_sink[head] * LOG2E;
  if (sk == CUDART_INF_F) return CUDART_INF_F;
  const float mx = fmaxf(a, sk);
  return mx + log2f(exp2f(a - mx) + exp2f(sk - mx));
}

struct BwdSmem {
  uint32_t q[HG * Q_W];
  uint32_t dout[HG * DO_W];
  uint32_t kv[TILE * KV_W];
  float p[HG * TILE];
  float ds[HG * TILE];
  float lse2[HG], delta[HG];
  int valid[TILE];
  int rowidx[TILE];
};

// Loads dO rows of a head group and returns nothing; delta[h] = sum_c O[h][c]*dO[h][c] is reduced by
// the 16 threads that share a head.
__device__ __forceinline__ void load_group_q_do(BwdSmem& s, const FmlaPrefillBwdArgs& a, int qi, int head0) {
  load_q_group(s.q, reinterpret_cast<const __nv_bfloat16*>(a.q) + qi * a.q_stride_s, a.q_stride_h, head0, a.h_q);
  const __nv_bfloat16* dop = reinterpret_cast<const __nv_bfloat16*>(a.dout) + qi * a.do_stride_s;
  for (int i = threadIdx.x; i < HG * 64; i += THREADS) {
    const int h = i / 64, c = i % 64;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (head0 + h < a.h_q) v = ldg_nc_16(dop + (head0 + h) * a.do_stride_h + 8 * c);
    *reinterpret_cast<uint4*>(s.dout + h * DO_W + 4 * c) = v;
  }
  // delta and lse: thread (h = tid/16, g = tid%16)
  const int h = threadIdx.x >> 4, g = threadIdx.x & 15, head = head0 + h;
  float d = 0.f;
  if (head < a.h_q) {
    const __nv_bfloat16* o = reinterpret_cast<const __nv_bfloat16*>(a.out) + ((int64_t)qi * a.h_q + head) * D_V;
    const __nv_bfloat16* dd = dop + head * a.do_stride_h;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 ov = ldg_nc_16(o + 8 * g + 128 * i), dv = ldg_nc_16(dd + 8 * g + 128 * i);
      d = dot_words(ov, dv, d);
    }
  }
#pragma unroll
  for (int off = 8; off; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
  if (g == 0) {
    s.delta[h] = d;
    s.lse2[h] = head < a.h_q ? lse_for_out_log2(a.lse[(int64_t)qi * a.h_q + head], a.attn_sink, head) : CUDART_INF_F;
  }
}

// Logit, P and dS of one (head, token): x = q.k*scale*log2e, P = 2^(x - lse2), dS = P*(dO.v - delta)*scale.
__device__ __forceinline__ void score_pair(const BwdSmem& s, int h, int j, float scale, float& p, float& ds) {
  const uint4* qp = reinterpret_cast<const uint4*>(s.q + h * Q_W);
  const uint4* dp_ = reinterpret_cast<const uint4*>(s.dout + h * DO_W);
  const uint4* kp = reinterpret_cast<const uint4*>(s.kv + j * KV_W);
  float x = 0.f, dp = 0.f;
#pragma unroll 4
  for (int c = 0; c < 64; ++c) {
    const uint4 kv = kp[c];
    x = dot_words(qp[c], kv, x);
    dp = dot_words(dp_[c], kv, dp);
  }
#pragma unroll
  for (int c = 64; c < 72; ++c) x = dot_words(qp[c], kp[c], x);
  p = s.valid[j] ? exp2f(x * scale * LOG2E - s.lse2[h]) : 0.f;
  ds = p * (dp - s.delta[h]) * scale;
}

// dQ: one block per (query, head group); thread (h, g) owns dq elements 4g + 64i + (0..3), i = 0..8.
__global__ void __launch_bounds__(THREADS)
prefill_bwd_dq_kernel(const FmlaPrefillBwdArgs a) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  BwdSmem& s = *reinterpret_cast<BwdSmem*>(smem_raw);
  const int qi = blockIdx.x, head0 = blockIdx.y * HG;
  const Bf16Rows rows{reinterpret_cast<const __nv_bfloat16*>(a.kv), a.kv_stride_s, a.s_kv, 72};
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  load_group_q_do(s, a, qi, head0);
  int limit = a.topk_length ? __ldg(a.topk_length + qi) : a.topk;
  limit = max(0, min(limit, a.topk));
  const int* idx = a.indices + qi * a.idx_stride_s;
  float acc[36];
#pragma unroll
  for (int e = 0; e < 36; ++e) acc[e] = 0.f;
  __syncthreads();
  for (int t0 = 0; t0 < limit; t0 += TILE) {
    {
      const int j = tid >> 3, sub = tid & 7, pos = t0 + j;
      const int id = pos < limit ? __ldg(idx + pos) : -1;
      const bool ok = rows.in_range(id);
      load_row(rows, id, ok, s.kv + j * KV_W, sub, 8);
      if (sub == 0) s.valid[j] = ok;
    }
    __syncthreads();
    {
      const int h = lane & 15, j0 = 4 * warp + (lane >> 4), j1 = j0 + 2;
      float p, ds;
      score_pair(s, h, j0, a.sm_scale, p, ds);
      s.ds[h * TILE + j0] = ds;
      score_pair(s, h, j1, a.sm_scale, p, ds);
      s.ds[h * TILE + j1] = ds;
    }
    __syncthreads();
    {
      const int h = tid >> 4, g = tid & 15;
      for (int j = 0; j < TILE; ++j) {
        const float ds = s.ds[h * TILE + j];
        const uint32_t* krow = s.kv + j * KV_W + 2 * g;
#pragma unroll
        for (int i = 0; i < 9; ++i) {
          const uint2 v = *reinterpret_cast<const uint2*>(krow + 32 * i);
          acc[4 * i + 0] = fmaf(ds, bf16_bits_to_float(v.x & 0xffffu), acc[4 * i + 0]);
          acc[4 * i + 1] = fmaf(ds, __uint_as_float(v.x & 0xffff0000u), acc[4 * i + 1]);
          acc[4 * i + 2] = fmaf(ds, bf16_bits_to_float(v.y & 0xffffu), acc[4 * i + 2]);
          acc[4 * i + 3] = fmaf(ds, __uint_as_float(v.y & 0xffff0000u), acc[4 * i + 3]);
        }
      }
    }
    __syncthreads();
  }
  const int h = tid >> 4, g = tid & 15, head = head0 + h;
  if (head < a.h_q) {
    __nv_bfloat16* dq = reinterpret_cast<__nv_bfloat16*>(a.dq) + ((int64_t)qi * a.h_q + head) * D_QK;
#pragma unroll
    for (int i = 0; i < 9; ++i)
      *reinterpret_cast<uint2*>(dq + 4 * g + 64 * i) =
          make_uint2(pack_bf16x2(acc[4 * i], acc[4 * i + 1]), pack_bf16x2(acc[4 * i + 2], acc[4 * i + 3]));
  }
}

// dKV: one block per query, all heads; per tile of 16 tokens thread (j = tid/16, g = tid%16) keeps the
// token's gradient elements 4g + 64i + (0..3) in registers across all head groups and issues one
// fp32 atomic add per element into dkv_accum[index[j]].
constexpr int TILE_B = 16;
__global__ void __launch_bounds__(THREADS)
prefill_bwd_dkv_kernel(const FmlaPrefillBwdArgs a) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  BwdSmem& s = *reinterpret_cast<BwdSmem*>(smem_raw);
  const int qi = blockIdx.x;
  const Bf16Rows rows{reinterpret_cast<const __nv_bfloat16*>(a.kv), a.kv_stride_s, a.s_kv, 72};
  const int tid = threadIdx.x;
  int limit = a.topk_length ? __ldg(a.topk_length + qi) : a.topk;
  limit = max(0, min(limit, a.topk));
  const int* idx = a.indices + qi * a.idx_stride_s;
  const int groups = (a.h_q + HG - 1) / HG;
  for (int t0 = 0; t0 < limit; t0 += TILE_B) {
    __syncthreads();
    {
      const int j = tid >> 4, sub = tid & 15, pos = t0 + j;
      const int id = pos < limit ? __ldg(idx + pos) : -1;
      const bool ok = rows.in_range(id);
      load_row(rows, id, ok, s.kv + j * KV_W, sub, 16);
      if (sub == 0) { s.valid[j] = ok; s.rowidx[j] = id; }
    }
    float acc_k[36], acc_v[32];
#pragma unroll
    for (int e = 0; e < 36; ++e) acc_k[e] = 0.f;
#pragma unroll
    for (int e = 0; e < 32; ++e) acc_v[e] = 0.f;
    for (int grp = 0; grp < groups; ++grp) {
      __syncthreads();
      load_group_q_do(s, a, qi, grp * HG);
      __syncthreads();
      {
        const int h = tid & 15, j = tid >> 4;
        float p, ds;
        score_pair(s, h, j, a.sm_scale, p, ds);
        s.p[h * TILE + j] = p;
        s.ds[h * TILE + j] = ds;
      }
      __syncthreads();
      {
        const int j = tid >> 4, g = tid & 15;
        for (int h = 0; h < HG; ++h) {
          const float ds = s.ds[h * TILE + j], p = s.p[h * TILE + j];
          const uint32_t* qrow = s.q + h * Q_W + 2 * g;
          const uint32_t* drow = s.dout + h * DO_W + 2 * g;
#pragma unroll
          for (int i = 0; i < 9; ++i) {
            const uint2 v = *reinterpret_cast<const uint2*>(qrow + 32 * i);
            acc_k[4 * i + 0] = fmaf(ds, bf16_bits_to_float(v.x & 0xffffu), acc_k[4 * i + 0]);
            acc_k[4 * i + 1] = fmaf(ds, __uint_as_float(v.x & 0xffff0000u), acc_k[4 * i + 1]);
            acc_k[4 * i + 2] = fmaf(ds, bf16_bits_to_float(v.y & 0xffffu), acc_k[4 * i + 2]);
            acc_k[4 * i + 3] = fmaf(ds, __uint_as_float(v.y & 0xffff0000u), acc_k[4 * i + 3]);
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint2 v = *reinterpret_cast<const uint2*>(drow + 32 * i);
            acc_v[4 * i + 0] = fmaf(p, bf16_bits_to_float(v.x & 0xffffu), acc_v[4 * i + 0]);
            acc_v[4 * i + 1] = fmaf(p, __uint_as_float(v.x & 0xffff0000u), acc_v[4 * i + 1]);
            acc_v[4 * i + 2] = fmaf(p, bf16_bits_to_float(v.y & 0xffffu), acc_v[4 * i + 2]);
            acc_v[4 * i + 3] = fmaf(p, __uint_as_float(v.y & 0xffff0000u), acc_v[4 * i + 3]);
          }
        }
      }
    }
    {
      const int j = tid >> 4, g = tid & 15;
      if (s.valid[j]) {
        float* dst = a.dkv_accum + (int64_t)s.rowidx[j] * D_QK + 4 * g;
#pragma unroll
        for (int i = 0; i < 9; ++i)
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            float v = acc_k[4 * i + k];
            if (i < 8) v += acc_v[4 * i + k];
            atomicAdd(dst + 64 * i + k, v);
          }
      }
    }
  }
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t n) {
  const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i + 3 < n) {
    const float4 v = *reinterpret_cast<const float4*>(src + i);
    *reinterpret_cast<uint2*>(dst + i) = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
  } else {
    for (int64_t k = i; k < n; ++k) dst[k] = __float2bfloat16_rn(src[k]);
  }
}

}  // namespace simt

template <class K>
static int set_smem(K kernel, size_t bytes) {
  FMLA_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  return FMLA_OK;
}

int launch_simt_decode(const FmlaDecodeArgs& a, cudaStream_t stream) {
  int plan_parts, overhead, block;
  if (int rc = fmla_decode_plan(a.device, a.h_q, a.s_q, FMLA_KERNEL_SIMT, &plan_parts, &overhead, &block)) return rc;
  dim3 grid(a.num_sm_parts, a.s_q, (a.h_q + simt::HG - 1) / simt::HG);
  if (a.layout == FMLA_LAYOUT_MODEL1) {
    if (int rc = set_smem(simt::decode_kernel<simt::PagedModel1Rows>, sizeof(simt::FwdSmem))) return rc;
    simt::decode_kernel<simt::PagedModel1Rows><<<grid, simt::THREADS, sizeof(simt::FwdSmem), stream>>>(a, block);
  } else {
    if (int rc = set_smem(simt::decode_kernel<simt::PagedFp8Rows>, sizeof(simt::FwdSmem))) return rc;
    simt::decode_kernel<simt::PagedFp8Rows><<<grid, simt::THREADS, sizeof(simt::FwdSmem), stream>>>(a, block);
  }
  FMLA_CUDA(cudaGetLastError());
  return FMLA_OK;
}

int launch_simt_prefill_fwd(const FmlaPrefillArgs& a, cudaStream_t stream) {
  if (int rc = set_smem(simt::prefill_fwd_kernel, sizeof(simt::FwdSmem))) return rc;
  dim3 grid(a.s_q, (a.h_q + simt::HG - 1) / simt::HG);
  simt::prefill_fwd_kernel<<<grid, simt::THREADS, sizeof(simt::FwdSmem), stream>>>(a);
  FMLA_CUDA(cudaGetLastError());
  return FMLA_OK;
}

int launch_simt_prefill_bwd(const FmlaPrefillBwdArgs& a, cudaStream_t stream) {
  FMLA_CUDA(cudaMemsetAsync(a.dkv_accum, 0, sizeof(float) * (size_t)a.s_kv * D_QK, stream));
  if (int rc = set_smem(simt::prefill_bwd_dq_kernel, sizeof(simt::BwdSmem))) return rc;
  if (int rc = set_smem(simt::prefill_bwd_dkv_kernel, sizeof(simt::BwdSmem))) return rc;
  dim3 grid(a.s_q, (a.h_q + simt::HG - 1) / simt::HG);
  simt::prefill_bwd_dq_kernel<<<grid, simt::THREADS, sizeof(simt::BwdSmem), stream>>>(a);
  FMLA_CUDA(cudaGetLastError());
  simt::prefill_bwd_dkv_kernel<<<a.s_q, simt::THREADS, sizeof(simt::BwdSmem), stream>>>(a);
  FMLA_CUDA(cudaGetLastError());
  if (a.dkv != nullptr) {
    const int64_t n = (int64_t)a.s_kv * D_QK;
    const int64_t blocks = (n / 4 + 255) / 256 + 1;
    simt::f32_to_bf16_kernel<<<(unsigned)blocks, 256, 0, stream>>>(a.dkv_accum, reinterpret_cast<__nv_bfloat16*>(a.dkv), n);
    FMLA_CUDA(cudaGetLastError());
  }
  return FMLA_OK;
}

}  // namespace fmla
