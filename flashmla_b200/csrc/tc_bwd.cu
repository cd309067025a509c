// Sparse prefill backward on the tcgen05 tensor cores (sm_100a), for head counts that are multiples of 64
// (a last group of 64 heads runs as a group of 128 whose upper half the TMA unit fills with zeros).
// The reference has no sparse backward (csrc/api/api.cpp:8-15 exports none); the mathematics follows its
// forward (tests/ref.py:19-52): with P = softmax over the selected tokens (and the sink) of q.k*sm_scale,
//     dP = dO V^T,  delta = rowsum(dO * O),  dS = P * (dP - delta) * sm_scale,
//     dQ = dS K,    dKV[idx] += dS^T Q  (all 576 dims)  +  P^T dO  (first 512 dims).
//
// A "unit" is one query token x one group of 128 heads: the M = 128 rows of every MMA.  The five products
// need 128 (S, dP) + 576 (dQ) + 576 (dKV) fp32 accumulator columns per unit, more than the 512 columns of
// tensor memory, so the work is cut into three kernels that hand P and dS over in bf16 through a caller-provided
// workspace ([units of a chunk][128 heads][topk rounded up to 128], 2 arrays):
//   bwd_scores_kernel  one CTA per unit.  Per block of 128 selected tokens: S = Q K^T and dP = dO V^T, both
//                      streamed over nine 64-wide feature chunks (Q chunk, dO chunk by TMA tile loads, K chunk by
//                      TMA gather4 of the indexed rows, one stage = 48 KB, 4 stages); S and dP are double-buffered
//                      in tensor memory (4 x 128 columns); four warps turn them into P and dS and store them.
//   dq_body            two CTAs per unit (feature panels 0-4 / 5-8).  dQ[128 x 320|256] += dS_blk [128 x 64] K_blk
//                      with K gathered as an MN-major B operand; one accumulator for the whole token list.
//   dkv_body           three CTAs per unit (192 features each).  Per block of 128 tokens D[128 tokens x 192] =
//                      dS^T Q + P^T dO with dS^T / P^T as MN-major A operands straight from the workspace tiles and
//                      Q / dO resident in shared memory; D is double-buffered in tensor memory and added to
//                      dkv_accum[idx] with 16-byte vector reductions (four lanes per row, 64 contiguous bytes).
// dq_body and dkv_body run as the five roles of one launch (bwd_dq_dkv_kernel), see there.
// Every kernel is warp-specialised the same way: warps 0-3 read tensor memory (warp w owns lanes 32w..32w+31),
// warp 4 issues the MMAs from one thread, the remaining warps issue TMA copies.  All waits are bounded and report
// through the status word instead of trapping.
#include <cuda.h>
#include <math_constants.h>

#include <algorithm>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "tensor_map.cuh"

namespace fmla {
namespace bwd {

using namespace ptx;

constexpr int HG = 128;                       // heads per unit
constexpr int NCHUNK = 9;                     // 64-wide feature panels of a 576-wide row
constexpr uint32_t TILE128 = 128 * 128;       // [128 rows x 64 bf16], 128-byte swizzled
constexpr uint32_t TILE64 = 64 * 128;         // [64 rows x 64 bf16]

// ---- TMA wrappers ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_gather4(uint32_t dst, const CUtensorMap* map, int col, int4 rows, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes.cta_group::1 [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
      ::"r"(dst), "l"(map), "r"(col), "r"(rows.x), "r"(rows.y), "r"(rows.z), "r"(rows.w), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_tile_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_tile_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void red_add_v4(float* dst, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(__uint_as_float(a)), "f"(__uint_as_float(b)),
               "f"(__uint_as_float(c)), "f"(__uint_as_float(d)) : "memory");
}
__device__ __forceinline__ uint4 lds_16(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
// 16 lanes x 32 columns as four 16x256b fragments: registers 4i..4i+3 belong to columns 8i..8i+7; lane t holds
// (row t/4, columns 2(t%4), 2(t%4)+1) in registers 4i, 4i+1 and (row t/4 + 8, same columns) in 4i+2, 4i+3.
__device__ __forceinline__ void tmem_ld_16x256b_x4(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x4.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void stg_16(void* dst, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// Streaming variants for the workspace, which is written once, read once by the next launch and far larger than
// L2: evict-first keeps it from pushing the KV rows (scores kernel) and the dKV rows (dQ/dKV kernel) out of L2.
__device__ __forceinline__ void stg_16_streaming(void* dst, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint64_t evict_first_policy() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void tma_tile_2d_hint(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar, uint64_t pol) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
               ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar), "l"(pol) : "memory");
}

// ---- parameters -------------------------------------------------------------------------------------------
struct Params {
  CUtensorMap map_q;      // q as (576, h_q, s_q): boxes of 64 dims x 128 heads
  CUtensorMap map_do;     // dout as (512, h_q, s_q): same boxes
  CUtensorMap map_kv;     // kv as (576, s_kv): one box = 64 dims of one row (gather4 takes four rows)
  CUtensorMap map_p;      // workspace P  as (topk_pad, chunk_units * 128): boxes of 64 slots x 128 heads
  CUtensorMap map_ds;     // workspace dS, same shape
  const int* indices; int64_t idx_stride_s;
  const int* topk_length;
  const float* lse; const float* attn_sink;
  const __nv_bfloat16* out; const __nv_bfloat16* dout; int64_t do_stride_s, do_stride_h;
  __nv_bfloat16* ws_p; __nv_bfloat16* ws_ds;
  __nv_bfloat16* dq; float* dkv_accum;
  int unit0;              // first unit of this chunk
  int groups;             // ceil(h_q / 128)
  int h_q, s_kv, topk, topk_pad;
  float sm_scale;
  int* status;
};

// ---- shared bookkeeping -----------------------------------------------------------------------------------
struct Ctx {
  uint32_t base;          // 1024-byte aligned start of the tiles
  uint32_t bars;          // first mbarrier
  volatile int* abort_flag;
  int* status;
};
__device__ __forceinline__ uint32_t bar_addr(const Ctx& c, int i) { return c.bars + 8u * i; }
__device__ __noinline__ void raise_abort(const Ctx& c, int code) {
  *c.abort_flag = code;
  if (c.status) atomicCAS(c.status, 0, code);
}
__device__ __forceinline__ bool wait(const Ctx& c, int bar, uint32_t parity, int code) {
  if (mbar_wait_abortable(bar_addr(c, bar), parity & 1u, c.abort_flag)) return true;
  if (*c.abort_flag == 0) raise_abort(c, code);
  return false;
}

struct Unit {
  int token, head0, local;
  int limit;              // number of index slots that count
  const int* idx;
};
__device__ __forceinline__ Unit get_unit(const Params& p, int local) {
  Unit u;
  u.local = local;
  const int g = p.unit0 + u.local;
  u.token = g / p.groups;
  u.head0 = (g - u.token * p.groups) * HG;
  int lim = p.topk_length ? __ldg(p.topk_length + u.token) : p.topk;
  u.limit = max(0, min(lim, p.topk));
  u.idx = p.indices + (int64_t)u.token * p.idx_stride_s;
  return u;
}
// Index of slot `pos`, or -1 when the slot does not count (the TMA unit zero-fills row -1).
__device__ __forceinline__ int slot_row(const Params& p, const Unit& u, int pos) {
  if (pos >= u.limit) return -1;
  const int id = __ldg(u.idx + pos);
  return (id >= 0 && id < p.s_kv) ? id : -1;
}

__device__ __forceinline__ float lse_with_sink_log2(float lse_nat, const float* attn_sink, int head) {
  if (lse_nat == CUDART_INF_F) return CUDART_INF_F;
  const float a = lse_nat * LOG2E;
  if (attn_sink == nullptr) return a;
  const float sk = attn_sink[head] * LOG2E;
  if (sk == CUDART_INF_F) return CUDART_INF_F;
  const float mx = fmaxf(a, sk);
  return mx + log2f(exp2f(a - mx) + exp2f(sk - mx));
}
__device__ __forceinline__ float dot_bf16x8(const uint4& a, const uint4& b, float acc) {
  const uint32_t x[4] = {a.x, a.y, a.z, a.w}, y[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc = fmaf(bf16_bits_to_float(x[i] & 0xffffu), bf16_bits_to_float(y[i] & 0xffffu), acc);
    acc = fmaf(__uint_as_float(x[i] & 0xffff0000u), __uint_as_float(y[i] & 0xffff0000u), acc);
  }
  return acc;
}

// Common prologue: carve shared memory, initialise `nbar` barriers with the given arrival counts, allocate
// tensor memory (warp 4).  Returns the tensor-memory base.
constexpr int MMA_WARP = 4;
__device__ __forceinline__ uint32_t prologue(Ctx& c, uint8_t* raw, uint32_t tile_bytes, const int* counts, int nbar, int* status) {
  const uint32_t raw_addr = smem_u32(raw);
  c.base = (raw_addr + 1023u) & ~1023u;
  const uint32_t ctl = c.base + tile_bytes;              // barriers | tmem word | abort word | scratch words
  c.bars = ctl;
  uint8_t* ctl_ptr = raw + (ctl - raw_addr);
  c.abort_flag = reinterpret_cast<volatile int*>(ctl_ptr + 8 * nbar + 4);
  c.status = status;
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    for (int i = 0; i < nbar; ++i) mbar_init(bar_addr(c, i), counts[i]);
    *c.abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == MMA_WARP) {
    tmem_alloc<1>(ctl + 8u * nbar, 512);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  return *reinterpret_cast<volatile uint32_t*>(ctl_ptr + 8 * nbar);
}
__device__ __forceinline__ void epilogue_dealloc(const Ctx& c, uint32_t tmem) {
  // A role that gave up on a wait leaves its loop with TMA copies possibly still in flight towards this CTA's
  // shared memory: give them a bounded time (64 us, far above a copy's latency) to land before the CTA exits.
  if (*c.abort_flag != 0)
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  tc_fence_before_sync();
  __syncthreads();
  if ((threadIdx.x >> 5) == MMA_WARP) {
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem, 512);
  }
}
constexpr uint32_t CTL_BYTES = 256;

// =============================================================================================================
// Kernel 1: P and dS
// =============================================================================================================
namespace sc {
constexpr int NST = 4;
constexpr uint32_t STAGE = 3 * TILE128;                 // Q chunk | dO chunk | K chunk
constexpr uint32_t TILES = NST * STAGE;
constexpr int NPROD = 8;                                // TMA-issuing warps
constexpr int THREADS = 32 * (5 + NPROD);
enum { FULL = 0, EMPTY = FULL + NST, S_FULL = EMPTY + NST, S_EMPTY = S_FULL + 2, NBAR = S_EMPTY + 2 };
constexpr uint32_t SMEM = TILES + CTL_BYTES + 1024;
}  // namespace sc

__global__ void __launch_bounds__(sc::THREADS, 1) bwd_scores_kernel(const __grid_constant__ Params p) {
  using namespace sc;
  extern __shared__ uint8_t smem_raw[];
  Ctx c;
  const int counts[NBAR] = {1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 128, 128};
  const uint32_t tmem = prologue(c, smem_raw, TILES, counts, NBAR, p.status);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const Unit u = get_unit(p, blockIdx.x);
  const int nblk = p.topk_pad / 128;

  if (warp < 4) {
    // ---- P / dS: thread = head row = tensor-memory lane
    const int row = threadIdx.x, head = u.head0 + row;
    const bool live = head < p.h_q;                        // rows past the last head: Q = dO = 0, P = dS = 0
    float delta = 0.f;
    if (live) {
      const __nv_bfloat16* o = p.out + ((int64_t)u.token * p.h_q + head) * D_V;
      const __nv_bfloat16* d = p.dout + (int64_t)u.token * p.do_stride_s + (int64_t)head * p.do_stride_h;
#pragma unroll 4
      for (int i = 0; i < D_V / 8; ++i) delta = dot_bf16x8(ldg_nc_16(o + 8 * i), ldg_nc_16(d + 8 * i), delta);
    }
    const float lse2 = live ? lse_with_sink_log2(p.lse[(int64_t)u.token * p.h_q + head], p.attn_sink, head) : CUDART_INF_F;
    const float scale2 = p.sm_scale * LOG2E;
    const uint32_t lane_base = tmem + ((uint32_t)(32 * warp) << 16);
    const int64_t ws_row = ((int64_t)u.local * HG + row) * p.topk_pad;
    // every warp derives a block's 128 validity bits itself; the indices behind them come from DRAM, so those of
    // the next block are requested before this block's accumulators are waited for
    uint32_t valid[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) valid[k] = __ballot_sync(0xffffffffu, slot_row(p, u, 32 * k + lane) >= 0);
    for (int blk = 0; blk < nblk; ++blk) {
      const int buf = blk & 1;
      int next_row[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) next_row[k] = blk + 1 < nblk ? slot_row(p, u, (blk + 1) * 128 + 32 * k + lane) : -1;
      if (!wait(c, S_FULL + buf, blk >> 1, 101)) break;
      tc_fence_after_sync();
#pragma unroll
      for (int piece = 0; piece < 4; ++piece) {
        uint32_t sv[32], dv[32];
        tmem_ld32(lane_base + 256 * buf + 32 * piece, sv);
        tmem_ld32(lane_base + 256 * buf + 128 + 32 * piece, dv);
        tmem_ld_wait();
        const uint32_t mask = valid[piece];
        uint32_t pp[16], dd[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          float p0 = exp2f(fmaf(__uint_as_float(sv[j]), scale2, -lse2));
          float p1 = exp2f(fmaf(__uint_as_float(sv[j + 1]), scale2, -lse2));
          if (!((mask >> j) & 1u)) p0 = 0.f;
          if (!((mask >> (j + 1)) & 1u)) p1 = 0.f;
          const float d0 = p0 * (__uint_as_float(dv[j]) - delta) * p.sm_scale;
          const float d1 = p1 * (__uint_as_float(dv[j + 1]) - delta) * p.sm_scale;
          pp[j >> 1] = pack_bf16x2(p0, p1);
          dd[j >> 1] = pack_bf16x2(d0, d1);
        }
        __nv_bfloat16* wp = p.ws_p + ws_row + blk * 128 + 32 * piece;
        __nv_bfloat16* wd = p.ws_ds + ws_row + blk * 128 + 32 * piece;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          stg_16_streaming(wp + 8 * k, pp[4 * k], pp[4 * k + 1], pp[4 * k + 2], pp[4 * k + 3]);
          stg_16_streaming(wd + 8 * k, dd[4 * k], dd[4 * k + 1], dd[4 * k + 2], dd[4 * k + 3]);
        }
      }
      tc_fence_before_sync();
      mbar_arrive(bar_addr(c, S_EMPTY + buf));
#pragma unroll
      for (int k = 0; k < 4; ++k) valid[k] = __ballot_sync(0xffffffffu, next_row[k] >= 0);
    }
  } else if (warp == MMA_WARP) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_bf16(128, 128, false, false);
      bool ok = true;
      for (int blk = 0; blk < nblk && ok; ++blk) {
        const int buf = blk & 1;
        if (blk >= 2 && !wait(c, S_EMPTY + buf, (blk >> 1) - 1, 102)) break;
        tc_fence_after_sync();
        for (int ch = 0; ch < NCHUNK; ++ch) {
          const int it = blk * NCHUNK + ch, st = it % NST;
          if (!wait(c, FULL + st, it / NST, 103)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t s0 = c.base + st * STAGE;
          const uint64_t aq = smem_desc_kmajor(s0), ad = smem_desc_kmajor(s0 + TILE128), bk = smem_desc_kmajor(s0 + 2 * TILE128);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) umma_ss<1>(tmem + 256 * buf, aq + 2 * ks, bk + 2 * ks, idesc, ch > 0 || ks > 0);
          if (ch < 8) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) umma_ss<1>(tmem + 256 * buf + 128, ad + 2 * ks, bk + 2 * ks, idesc, ch > 0 || ks > 0);
          }
          umma_commit<1>(bar_addr(c, EMPTY + st), 0);
        }
        if (ok) umma_commit<1>(bar_addr(c, S_FULL + buf), 0);
      }
    }
  } else {
    // ---- producers.  A warp whose 32 lanes each issue a gather4 was measured busy for 3.8 k cycles per stage; with
    // the 34 operations of a stage spread over NPROD warps each warp is busy 1.1 k cycles, so every stage is filled
    // by all of them together: warp pw gathers rows 16 pw .. 16 pw + 15 (four lanes), warp 0 also sets the stage's
    // byte count and loads the Q and dO chunks.
    const int pw = warp - 5;
    const int total = nblk * NCHUNK;
    auto rows_of = [&](int blk) {
      const int pos = blk * 128 + 16 * pw + 4 * (lane & 3);
      return make_int4(slot_row(p, u, pos), slot_row(p, u, pos + 1), slot_row(p, u, pos + 2), slot_row(p, u, pos + 3));
    };
    int4 rows = rows_of(0), next_rows = rows;
    for (int it = 0; it < total; ++it) {
      const int blk = it / NCHUNK, ch = it - blk * NCHUNK, st = it % NST;
      const uint32_t use = it / NST;
      if (ch == 0) {                                       // the next block's indices are requested a block ahead
        rows = next_rows;
        if (blk + 1 < nblk) next_rows = rows_of(blk + 1);
      }
      bool ok = use == 0 || wait(c, EMPTY + st, use - 1, 104);
      if (!__all_sync(0xffffffffu, ok)) break;
      const uint32_t s0 = c.base + st * STAGE, bar = bar_addr(c, FULL + st);
      if (pw == 0 && lane == 0) {
        mbar_expect_tx(bar, (ch < 8 ? 3u : 2u) * TILE128);
        tma_tile_3d(s0, &p.map_q, 64 * ch, u.head0, u.token, bar);
        if (ch < 8) tma_tile_3d(s0 + TILE128, &p.map_do, 64 * ch, u.head0, u.token, bar);
      }
      if (lane < 4) tma_gather4(s0 + 2 * TILE128 + 512u * (4 * pw + lane), &p.map_kv, 64 * ch, rows, bar);
    }
  }
  epilogue_dealloc(c, tmem);
}

// =============================================================================================================
// Kernel 2: dQ
// =============================================================================================================
namespace dqk {
constexpr int NST = 3;
constexpr uint32_t STAGE = TILE128 + 5 * TILE64;        // dS tile [128 heads x 64 slots] | up to 5 K panels [64 slots x 64 dims]
constexpr uint32_t TILES = NST * STAGE;
constexpr int NPROD = 8;                                // TMA-issuing warps
constexpr int THREADS = 32 * (5 + NPROD);
enum { FULL = 0, EMPTY = FULL + NST, DONE = EMPTY + NST, NBAR = DONE + 1 };
constexpr uint32_t SMEM = TILES + CTL_BYTES + 1024;
}  // namespace dqk

__device__ __forceinline__ void dq_body(const Params& p, uint8_t* smem_raw, int local, int half) {
  using namespace dqk;
  Ctx c;
  const int counts[NBAR] = {1, 1, 1, 1, 1, 1, 1};
  const uint32_t tmem = prologue(c, smem_raw, TILES, counts, NBAR, p.status);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const Unit u = get_unit(p, local);
  const int nblk = p.topk_pad / 64;
  const int panel0 = half == 0 ? 0 : 5, npan = half == 0 ? 5 : 4;

  if (warp < 4) {
    const int row = threadIdx.x;
    const uint32_t lane_base = tmem + ((uint32_t)(32 * warp) << 16);
    if (wait(c, DONE, 0, 111) && u.head0 + row < p.h_q) {
      tc_fence_after_sync();
      __nv_bfloat16* dst = p.dq + ((int64_t)u.token * p.h_q + u.head0 + row) * D_QK + 64 * panel0;
#pragma unroll 1
      for (int piece = 0; piece < 2 * npan; ++piece) {
        uint32_t v[32];
        tmem_ld32(lane_base + 32 * piece, v);
        tmem_ld_wait();
#pragma unroll
        for (int k = 0; k < 4; ++k)
          stg_16(dst + 32 * piece + 8 * k, pack_bf16x2(__uint_as_float(v[8 * k]), __uint_as_float(v[8 * k + 1])),
                 pack_bf16x2(__uint_as_float(v[8 * k + 2]), __uint_as_float(v[8 * k + 3])),
                 pack_bf16x2(__uint_as_float(v[8 * k + 4]), __uint_as_float(v[8 * k + 5])),
                 pack_bf16x2(__uint_as_float(v[8 * k + 6]), __uint_as_float(v[8 * k + 7])));
      }
    }
  } else if (warp == MMA_WARP) {
    if (lane == 0) {
      constexpr uint32_t idesc256 = idesc_bf16(128, 256, false, true), idesc64 = idesc_bf16(128, 64, false, true);
      bool ok = true;
      for (int it = 0; it < nblk; ++it) {
        const int st = it % NST;
        if (!wait(c, FULL + st, it / NST, 112)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t s0 = c.base + st * STAGE;
        const uint64_t a = smem_desc_kmajor(s0), b = smem_desc_mnmajor(s0 + TILE128, TILE64);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          umma_ss<1>(tmem, a + 2 * ks, b + ((ks * 2048) >> 4), idesc256, it > 0 || ks > 0);
          if (npan == 5) umma_ss<1>(tmem + 256, a + 2 * ks, b + ((4 * TILE64 + ks * 2048) >> 4), idesc64, it > 0 || ks > 0);
        }
        umma_commit<1>(bar_addr(c, EMPTY + st), 0);
      }
      if (ok) umma_commit<1>(bar_addr(c, DONE), 0);
    }
  } else if (warp < 5 + NPROD) {
    // all NPROD warps fill every stage together (see the scores kernel): warp pw gathers row groups 2 pw and
    // 2 pw + 1 of the 64 slots, one lane per (row group, feature panel); warp 0 also loads the dS tile
    const int pw = warp - 5;
    const int grp = 2 * pw + lane / npan, pn = lane % npan;
    const bool active = lane < 2 * npan;
    auto rows_of = [&](int it) {
      const int pos = it * 64 + 4 * grp;
      return make_int4(slot_row(p, u, pos), slot_row(p, u, pos + 1), slot_row(p, u, pos + 2), slot_row(p, u, pos + 3));
    };
    int4 rows = active ? rows_of(0) : make_int4(-1, -1, -1, -1);
    for (int it = 0; it < nblk; ++it) {
      const int st = it % NST;
      const uint32_t use = it / NST;
      bool ok = use == 0 || wait(c, EMPTY + st, use - 1, 113);
      if (!__all_sync(0xffffffffu, ok)) break;
      const uint32_t s0 = c.base + st * STAGE, bar = bar_addr(c, FULL + st);
      if (pw == 0 && lane == 0) {
        mbar_expect_tx(bar, TILE128 + npan * TILE64);
        tma_tile_2d_hint(s0, &p.map_ds, 64 * it, u.local * HG, bar, evict_first_policy());
      }
      if (active) {
        tma_gather4(s0 + TILE128 + pn * TILE64 + 512u * grp, &p.map_kv, 64 * (panel0 + pn), rows, bar);
        if (it + 1 < nblk) rows = rows_of(it + 1);         // indices of the next stage, fresh from DRAM, one use ahead
      }
    }
  }
  epilogue_dealloc(c, tmem);
}

// =============================================================================================================
// Kernel 3: dKV
// =============================================================================================================
namespace dkvk {
constexpr int NST = 2;
constexpr uint32_t RES = 6 * TILE128;                   // Q panels (3) | dO panels (up to 3), [128 heads x 64 dims] each
constexpr uint32_t STAGE = 4 * TILE128;                 // dS tiles for slots 0-63, 64-127 | P tiles likewise
constexpr uint32_t TILES = RES + NST * STAGE;
constexpr int THREADS = 32 * 6;
enum { FULL = 0, EMPTY = FULL + NST, D_FULL = EMPTY + NST, D_EMPTY = D_FULL + 2, RES_FULL = D_EMPTY + 2, RES_READY, NBAR };
constexpr uint32_t SMEM = TILES + CTL_BYTES + 1024;
static_assert(SMEM <= 227 * 1024, "shared memory budget exceeded");
}  // namespace dkvk

__device__ __forceinline__ void dkv_body(const Params& p, uint8_t* smem_raw, int local, int third) {
  using namespace dkvk;
  Ctx c;
  const int counts[NBAR] = {1, 1, 1, 1, 1, 1, 128, 128, 1, 128};
  const uint32_t tmem = prologue(c, smem_raw, TILES, counts, NBAR, p.status);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const Unit u = get_unit(p, local);
  const int nblk = p.topk_pad / 128;                     // this CTA's features: [192 third, 192 third + 192)
  const int nv = third < 2 ? 3 : 2;                      // dO panels in range (features below 512)

  if (warp < 4) {
    const uint32_t lane_base = tmem + ((uint32_t)(32 * warp) << 16);
    // The 16x256b tensor-memory reads below hand a lane two adjacent columns per 8-column fragment.  The resident
    // Q / dO tiles are re-ordered once, inside every group of 16 features, so that accumulator column 8i + 2m + e
    // of a group holds feature 4m + 2i + e: the two fragments of a group then give lane m four consecutive features,
    // one 16-byte reduction instead of two 8-byte ones.
    if (wait(c, RES_FULL, 0, 126)) {
      const uint32_t r = threadIdx.x;
      for (int t = 0; t < 3 + nv; ++t)
#pragma unroll
        for (uint32_t cp = 0; cp < 8; cp += 2) {
          const uint32_t a0 = c.base + t * TILE128 + swz(r, cp), a1 = c.base + t * TILE128 + swz(r, cp + 1);
          const uint4 v0 = lds_16(a0), v1 = lds_16(a1);
          st_shared16(a0, make_uint4(v0.x, v0.z, v1.x, v1.z));
          st_shared16(a1, make_uint4(v0.y, v0.w, v1.y, v1.w));
        }
      fence_async_smem();
      mbar_arrive(bar_addr(c, RES_READY));
    }
    int next_id = slot_row(p, u, threadIdx.x);
    for (int blk = 0; blk < nblk; ++blk) {
      const int buf = blk & 1;
      const int id = next_id;                              // looked up one block ahead: the indices come from DRAM
      next_id = blk + 1 < nblk ? slot_row(p, u, (blk + 1) * 128 + threadIdx.x) : -1;
      if (!wait(c, D_FULL + buf, blk >> 1, 121)) break;
      tc_fence_after_sync();
      // 16x256b reads: lane t receives, per 8-column fragment, rows t/4 and t/4 + 8 of a 16-row window at columns
      // 2 (t%4) and 2 (t%4) + 1; with the feature order set up above two fragments give the lane four consecutive
      // features, so the four lanes of a row cover 64 contiguous bytes and a warp instruction eight rows.
      const int ids[4] = {__shfl_sync(0xffffffffu, id, lane >> 2), __shfl_sync(0xffffffffu, id, (lane >> 2) + 8),
                          __shfl_sync(0xffffffffu, id, (lane >> 2) + 16), __shfl_sync(0xffffffffu, id, (lane >> 2) + 24)};
      float* col0 = p.dkv_accum + 192 * third + 4 * (lane & 3);
#pragma unroll 1
      for (int piece = 0; piece < 6; ++piece) {
        uint32_t lo[16], hi[16];
        tmem_ld_16x256b_x4(lane_base + 256 * buf + 32 * piece, lo);                    // rows 0-15 of this warp's window
        tmem_ld_16x256b_x4(lane_base + (16u << 16) + 256 * buf + 32 * piece, hi);      // rows 16-31
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 2; ++g) {                      // fragments 2g, 2g+1 = features 16g + 4 (lane % 4) .. + 3
          const int col = 32 * piece + 16 * g;
          const int f0 = 8 * g, f1 = 8 * g + 4;
          if (ids[0] >= 0) red_add_v4(col0 + (int64_t)ids[0] * D_QK + col, lo[f0], lo[f0 + 1], lo[f1], lo[f1 + 1]);
          if (ids[1] >= 0) red_add_v4(col0 + (int64_t)ids[1] * D_QK + col, lo[f0 + 2], lo[f0 + 3], lo[f1 + 2], lo[f1 + 3]);
          if (ids[2] >= 0) red_add_v4(col0 + (int64_t)ids[2] * D_QK + col, hi[f0], hi[f0 + 1], hi[f1], hi[f1 + 1]);
          if (ids[3] >= 0) red_add_v4(col0 + (int64_t)ids[3] * D_QK + col, hi[f0 + 2], hi[f0 + 3], hi[f1 + 2], hi[f1 + 3]);
        }
      }
      tc_fence_before_sync();
      mbar_arrive(bar_addr(c, D_EMPTY + buf));
    }
  } else if (warp == MMA_WARP) {
    if (lane == 0) {
      constexpr uint32_t idesc192 = idesc_bf16(128, 192, true, true), idesc128 = idesc_bf16(128, 128, true, true);
      const uint32_t idesc_v = nv == 3 ? idesc192 : idesc128;
      bool ok = wait(c, RES_READY, 0, 122);
      const uint64_t bq = smem_desc_mnmajor(c.base, TILE128), bd = smem_desc_mnmajor(c.base + 3 * TILE128, TILE128);
      for (int blk = 0; blk < nblk && ok; ++blk) {
        const int buf = blk & 1, st = blk % NST;
        if (blk >= 2 && !wait(c, D_EMPTY + buf, (blk >> 1) - 1, 123)) break;
        if (!wait(c, FULL + st, blk / NST, 124)) break;
        tc_fence_after_sync();
        const uint32_t s0 = c.base + RES + st * STAGE;
        const uint64_t ads = smem_desc_mnmajor(s0, TILE128), ap = smem_desc_mnmajor(s0 + 2 * TILE128, TILE128);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ss<1>(tmem + 256 * buf, ads + ((ks * 2048) >> 4), bq + ((ks * 2048) >> 4), idesc192, ks > 0);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ss<1>(tmem + 256 * buf, ap + ((ks * 2048) >> 4), bd + ((ks * 2048) >> 4), idesc_v, true);
        umma_commit<1>(bar_addr(c, EMPTY + st), 0);
        umma_commit<1>(bar_addr(c, D_FULL + buf), 0);
      }
    }
  } else if (warp == MMA_WARP + 1) {
    if (lane == 0) {
      const uint32_t rbar = bar_addr(c, RES_FULL);
      mbar_expect_tx(rbar, (3 + nv) * TILE128);
      for (int k = 0; k < 3; ++k) tma_tile_3d(c.base + k * TILE128, &p.map_q, 192 * third + 64 * k, u.head0, u.token, rbar);
      for (int k = 0; k < nv; ++k) tma_tile_3d(c.base + (3 + k) * TILE128, &p.map_do, 192 * third + 64 * k, u.head0, u.token, rbar);
      for (int blk = 0; blk < nblk; ++blk) {
        const int st = blk % NST;
        const uint32_t use = blk / NST;
        if (use > 0 && !wait(c, EMPTY + st, use - 1, 125)) break;
        const uint32_t s0 = c.base + RES + st * STAGE, bar = bar_addr(c, FULL + st);
        mbar_expect_tx(bar, STAGE);
        const uint64_t pol = evict_first_policy();
        tma_tile_2d_hint(s0, &p.map_ds, 128 * blk, u.local * HG, bar, pol);
        tma_tile_2d_hint(s0 + TILE128, &p.map_ds, 128 * blk + 64, u.local * HG, bar, pol);
        tma_tile_2d_hint(s0 + 2 * TILE128, &p.map_p, 128 * blk, u.local * HG, bar, pol);
        tma_tile_2d_hint(s0 + 3 * TILE128, &p.map_p, 128 * blk + 64, u.local * HG, bar, pol);
      }
    }
  }
  epilogue_dealloc(c, tmem);
}

// One launch for both: CTAs (unit, 0..2) are the dKV thirds, (unit, 3..4) the dQ halves, with the role as the fast
// grid dimension so that both kinds are resident at any time.  The dKV CTAs are bound by the rate at which L2
// takes fp32 reductions (about 3 TB/s on the whole chip, whatever the instruction mix) and leave the tensor
// cores idle most of the time; the dQ CTAs need no reductions, so the two overlap instead of adding up.
constexpr int GRAD_ROLES = 5;
constexpr int GRAD_THREADS = dqk::THREADS > dkvk::THREADS ? dqk::THREADS : dkvk::THREADS;
constexpr uint32_t GRAD_SMEM = dqk::SMEM > dkvk::SMEM ? dqk::SMEM : dkvk::SMEM;
__global__ void __launch_bounds__(GRAD_THREADS, 1) bwd_dq_dkv_kernel(const __grid_constant__ Params p) {
  extern __shared__ uint8_t smem_raw[];
  const int role = blockIdx.x, local = blockIdx.y;
  if (role < 3) dkv_body(p, smem_raw, local, role);
  else dq_body(p, smem_raw, local, role - 3);
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

// ---- host -------------------------------------------------------------------------------------------------
// bf16 tensor of `rank` dims (innermost first) with byte strides for dims 1.., 128-byte swizzled boxes.
static int make_map(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides,
                    const uint32_t* box, const char* what) {
  const int rc = tmap::encode(map, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  FMLA_REQUIRE(rc >= 0, FMLA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  FMLA_REQUIRE(rc == 0, FMLA_ERR_CUDA, "sparse_prefill_bwd: cuTensorMapEncodeTiled failed for %s with driver error %d", what, rc);
  return FMLA_OK;
}

}  // namespace bwd

bool tc_bwd_supported(int h_q) { return h_q > 0 && h_q % 64 == 0; }
int tc_bwd_groups(int h_q) { return (h_q + bwd::HG - 1) / bwd::HG; }

int64_t tc_bwd_unit_bytes(int topk) {
  const int64_t topk_pad = ((int64_t)topk + 127) / 128 * 128;
  return 2 * (int64_t)bwd::HG * topk_pad * 2;
}

int launch_tc_prefill_bwd(const FmlaPrefillBwdArgs& a, cudaStream_t stream) {
  using namespace bwd;
  FMLA_REQUIRE(tc_bwd_supported(a.h_q), FMLA_ERR_UNSUPPORTED, "sparse_prefill_bwd: the tensor-core kernels need h_q to be a multiple of 64 (got %d)", a.h_q);
  const int64_t unit_bytes = tc_bwd_unit_bytes(a.topk);
  FMLA_REQUIRE(a.workspace != nullptr && a.workspace_bytes >= unit_bytes && (reinterpret_cast<uintptr_t>(a.workspace) & 127u) == 0,
               FMLA_ERR_INVALID_ARG,
               "sparse_prefill_bwd: the tensor-core kernels need a 128-byte aligned workspace of at least %lld bytes (got %lld)",
               (long long)unit_bytes, (long long)a.workspace_bytes);
  const int groups = tc_bwd_groups(a.h_q);
  const int64_t units = (int64_t)a.s_q * groups;
  const int64_t chunk = std::min<int64_t>(units, std::min<int64_t>(a.workspace_bytes / unit_bytes, 65535));   // units are a grid y dimension
  const int topk_pad = (a.topk + 127) / 128 * 128;

  Params p{};
  {
    const uint64_t dims[3] = {(cuuint64_t)D_QK, (cuuint64_t)a.h_q, (cuuint64_t)a.s_q};
    const uint64_t strides[2] = {(cuuint64_t)a.q_stride_h * 2, (cuuint64_t)a.q_stride_s * 2};
    const uint32_t box[3] = {64, HG, 1};
    if (int rc = make_map(&p.map_q, a.q, 3, dims, strides, box, "q")) return rc;
  }
  {
    const uint64_t dims[3] = {(cuuint64_t)D_V, (cuuint64_t)a.h_q, (cuuint64_t)a.s_q};
    const uint64_t strides[2] = {(cuuint64_t)a.do_stride_h * 2, (cuuint64_t)a.do_stride_s * 2};
    const uint32_t box[3] = {64, HG, 1};
    if (int rc = make_map(&p.map_do, a.dout, 3, dims, strides, box, "dout")) return rc;
  }
  {
    const uint64_t dims[2] = {(cuuint64_t)D_QK, (cuuint64_t)a.s_kv};
    const uint64_t strides[1] = {(cuuint64_t)a.kv_stride_s * 2};
    const uint32_t box[2] = {64, 1};
    if (int rc = make_map(&p.map_kv, a.kv, 2, dims, strides, box, "kv")) return rc;
  }
  __nv_bfloat16* ws_p = static_cast<__nv_bfloat16*>(a.workspace);
  __nv_bfloat16* ws_ds = ws_p + chunk * HG * topk_pad;
  {
    const uint64_t dims[2] = {(cuuint64_t)topk_pad, (cuuint64_t)(chunk * HG)};
    const uint64_t strides[1] = {(cuuint64_t)topk_pad * 2};
    const uint32_t box[2] = {64, HG};
    if (int rc = make_map(&p.map_p, ws_p, 2, dims, strides, box, "workspace")) return rc;
    if (int rc = make_map(&p.map_ds, ws_ds, 2, dims, strides, box, "workspace")) return rc;
  }
  p.indices = a.indices; p.idx_stride_s = a.idx_stride_s; p.topk_length = a.topk_length;
  p.lse = a.lse; p.attn_sink = a.attn_sink;
  p.out = static_cast<const __nv_bfloat16*>(a.out); p.dout = static_cast<const __nv_bfloat16*>(a.dout);
  p.do_stride_s = a.do_stride_s; p.do_stride_h = a.do_stride_h;
  p.ws_p = ws_p; p.ws_ds = ws_ds;
  p.dq = static_cast<__nv_bfloat16*>(a.dq); p.dkv_accum = a.dkv_accum;
  p.groups = groups; p.h_q = a.h_q; p.s_kv = a.s_kv; p.topk = a.topk; p.topk_pad = topk_pad;
  p.sm_scale = a.sm_scale; p.status = a.status;

  static tmap::PerDeviceOnce once;
  FMLA_CUDA(once.run([] {
    const cudaError_t e = cudaFuncSetAttribute(bwd_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sc::SMEM);
    return e != cudaSuccess ? e : cudaFuncSetAttribute(bwd_dq_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GRAD_SMEM);
  }));
  FMLA_CUDA(cudaMemsetAsync(a.dkv_accum, 0, sizeof(float) * (size_t)a.s_kv * D_QK, stream));
  for (int64_t u0 = 0; u0 < units; u0 += chunk) {
    const unsigned n = (unsigned)std::min<int64_t>(chunk, units - u0);
    p.unit0 = (int)u0;
    bwd_scores_kernel<<<n, sc::THREADS, sc::SMEM, stream>>>(p);
    FMLA_CUDA(cudaGetLastError());
    const bool timed = u0 == 0 && a.grad_begin_event != nullptr && a.grad_end_event != nullptr;
    if (timed) FMLA_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(a.grad_begin_event), stream));
    bwd_dq_dkv_kernel<<<dim3(GRAD_ROLES, n), GRAD_THREADS, GRAD_SMEM, stream>>>(p);
    FMLA_CUDA(cudaGetLastError());
    if (timed) FMLA_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(a.grad_end_event), stream));
  }
  if (a.dkv != nullptr) {
    const int64_t n = (int64_t)a.s_kv * D_QK;
    const int64_t blocks = (n / 4 + 255) / 256 + 1;
    f32_to_bf16_kernel<<<(unsigned)blocks, 256, 0, stream>>>(a.dkv_accum, static_cast<__nv_bfloat16*>(a.dkv), n);
    FMLA_CUDA(cudaGetLastError());
  }
  return FMLA_OK;
}

}  // namespace fmla
