// Tensor-core (tcgen05) sparse MLA attention: decode over the paged FP8 / MXFP8 cache (optionally over two
// caches) and sparse prefill forward are instantiations of one persistent kernel.
//
// A cluster of two CTAs (a "pair", tcgen05 cta_group::2) owns 128 heads of one query at a time (a last group of
// 64 heads runs with its upper half padded by zero queries): CTA r keeps heads [64r, 64r+64) and, of every
// gathered KV row, only one half of the feature dimension:
//     half 0 = NoPE[0:256]   + RoPE[0:32],     half 1 = NoPE[256:512] + RoPE[32:64]   (288 dims each)
// so every row is fetched and dequantised exactly once per pair.  Work is cut into blocks of T = 64 token slots, and a
// block passes through these roles (warps per CTA):
//
//   prefill producers (8)    warp w owns tokens [8w, 8w+8): indices prefetched into a shared-memory ring by
//                            cp.async, rows gathered with cp.async.bulk.tensor tile::gather4 (four rows per
//                            instruction, one instruction per lane) straight into the stage: four 128B-swizzled
//                            NoPE panels [64 tokens x 64 dims] and one 64B-swizzled RoPE panel [64 x 32].  An
//                            invalid slot gets row coordinate -1, which the TMA unit zero-fills.  The gathers
//                            signal the leader CTA's stage barrier themselves.
//   decode gather (4)        warp g fetches rows [16g, 16g+16) into a two-slot raw ring: per four rows one gather of
//                            256 bytes a row (this CTA's NoPE half), one of 64 (its RoPE half) and one of 16 (scales).
//   decode convert (8)       each dequantises eight rows of the raw slot into the stage: e4m3x2 -> f16x2 (one
//                            cvt, exact) times the tile scale as f16x2.  Every e4m3 value times a power-of-two
//                            scale up to 2^7 is exact in fp16 (|x| <= 448 * 128 = 57344 < 65504); larger scales
//                            saturate at 2^7 and are reported through the status word.  RoPE stays bf16.
//   QK^T  (2 threads, CTA 0) S = Q K^T of a block is 20 x tcgen05.mma M=128 N=128 K=16 into one of two S buffers in
//                            tensor memory; the two issuers take alternate blocks.  16 NoPE k-steps: A = Q from tensor
//                            memory, B = the stage (K-major), f16 x f16 in decode (Q is converted once per item), bf16 x
//                            bf16 in prefill.  N-half 0 comes from CTA 0's stage (feature half 0), N-half 1 from CTA 1's
//                            (half 1); the A operand is lane-local, lanes 0-63 hold Q[:, half 0] and lanes 64-127
//                            Q[:, half 1], so lanes 0-63 / 64-127 of the accumulator receive the two partial dot
//                            products of the same 64 heads x 64 tokens.  The RoPE part of Q lives in shared memory
//                            (tensor memory is full): its 2 k-steps are 4 products with the lanes of the other feature
//                            half masked off (disable-output-lane).
//   softmax (8, two teams)   team t (four warps, one per quarter of the tensor-memory lanes) takes the blocks of parity
//                            t, so two blocks are in flight.  The two threads of a head in a team (the two feature
//                            halves) add their partials through shared memory, apply the validity mask, run the online
//                            softmax in base 2 and write P (f16 in decode, bf16 in prefill) as the A operand of PV.
//                            The reference maximum moves lazily and is handed from team to team, block by block.  The
//                            softmax warps also move each query's Q into tensor memory and run the epilogue.
//   PV    (1 thread, CTA 0)  8 x tcgen05.mma M=128 N=256 K=16, A = P (shared memory, K-major), B = the same
//                            stage viewed MN-major: CTA r's four NoPE panels are exactly V[:, 256r:256r+256].
//                            O accumulates in tensor memory: lanes 0-63 = O[:, 0:256], lanes 64-127 = O[:, 256:512].
//
// Tensor memory (512 columns): O 0-255 | Q (NoPE) 256-383 | S buffers 384-447, 448-511.
//
// The stages form a ring used in a fixed order of positions.  The two positions before an item's first block carry the
// item's Q, fetched by the stage-filling warps as far ahead as the KV rows (fill_q_positions); at the end of the item
// before, the softmax warps copy it into tensor memory - the idle team while the last block's softmax still runs - and
// the next item's first QK^T products overlap the last PV product and the epilogue.
//
// All cross-role hand-offs are mbarriers; every wait is bounded and a time-out raises an abort flag, sets *status and
// lets all roles fall through to the teardown.  A shared-memory buffer that changes hands between generic-proxy
// accesses and TMA writes is fenced with fence.proxy.async on the generic side before the barrier that hands it over.
//
// The kernel is persistent: a pair walks a list of work items - for decode the (request, block range)
// pieces its tile-scheduler record assigns, for prefill every n-th query token - and the producers and
// MMA issuers run ahead across item boundaries.
//
// Numerics follow the reference's oracle (tests/ref.py:19-103): natural-log lse over valid slots, out = 0
// and lse = +inf for a query without valid slot, attn_sink rescales out only; P is rounded to 16 bits before
// PV while the row sum uses the unrounded values, like the reference's kernels
// (csrc/sm100/prefill/sparse/common_subroutine.h:186-206).
#include <cuda.h>

#include <atomic>
#include <math_constants.h>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "tensor_map.cuh"

namespace fmla {
namespace tc {
using namespace ptx;

constexpr int T = 64;                 // index slots per block
constexpr int NPW = 8;                // producer warps per CTA
constexpr int PROWS = 64 / NPW;       // tokens of a block owned by one producer warp
constexpr int NSW = 8;                // softmax warps per CTA: two teams of four (one warp per quarter of the tensor-memory lanes)
constexpr int NGW = 4;                // decode: gather warps, each fetching 16 of a block's 64 rows
constexpr int GROWS = 64 / NGW;       // rows of a block fetched by one gather warp
// warps: NSW softmax, NPW producers / converters, two QK^T issuers (one per S buffer), the PV issuer and an idle warp,
// NGW gather warps (decode only)
constexpr int QK_WARP = NSW + NPW, PV_WARP = QK_WARP + 2, GATHER_WARP = QK_WARP + 4;
// decode runs all warps; prefill has no gather warps (24 / 20 warps)
// FP8 decode (variants 0-2) passes its rows through the raw ring: gather warps fetch, converter warps dequantise.
// Prefill and dense decode (variant 3) gather bf16 rows straight into the stages.
constexpr bool raw_ring(int mode, int variant) { return mode == 0 && variant != 3; }
constexpr int threads_of(bool raw) { return 32 * (GATHER_WARP + (raw ? NGW : 0)); }
constexpr int NSTAGE_DECODE = 4, NSTAGE_PREFILL = 5, NRAW = 2, MAX_STAGES = 5;
constexpr uint32_t PANEL = T * 128;                 // one 128B-swizzled [64 tokens x 64 dims] panel
constexpr uint32_t ROPE_PANEL = 4 * PANEL;          // offset of the 64B-swizzled [64 x 32] RoPE panel in a stage
constexpr uint32_t STAGE_BYTES = 4 * PANEL + T * 64;
constexpr uint32_t STAGE_TX_BYTES = T * (512 + 64);
// raw slot (decode): 64 rows x 256 NoPE bytes of this CTA's feature half; then per group of four rows the rows' 16-byte
// scale fields (bytes 512..527) and this CTA's 64-byte RoPE halves; groups are spaced so that every gather destination
// is 128-byte aligned
constexpr uint32_t RAW_NOPE = 0, RAW_SCALE = T * 256, SCALE_GROUP = 128, RAW_ROPE = RAW_SCALE + (T / 4) * SCALE_GROUP, ROPE_GROUP = 256;
constexpr uint32_t RAW_BYTES = (RAW_ROPE + (T / 4) * ROPE_GROUP + 1023) / 1024 * 1024;
constexpr uint32_t RAW_TX_BYTES = GROWS * (256 + 16 + 64);      // bytes one gather warp brings per block
// raw slot, MODEL1 (d_qk = 512: a row is 448 e4m3 + 64 bf16, and CTA r owns values [256r, 256r+256) of it): CTA 0 holds
// 64 rows x 256 e4m3 bytes, CTA 1 64 rows x 192 e4m3 bytes and then 64 rows x 128 bytes of bf16; then, in both, the rows'
// eight scale bytes (seven e8m0, one per 64 values), which the gather warps fetch with plain loads
constexpr uint32_t M1_RAW_ROPE = T * 192, M1_RAW_SCALE = M1_RAW_ROPE + T * 128;
static_assert(M1_RAW_SCALE + T * 8 <= RAW_BYTES && M1_RAW_SCALE >= T * 256, "MODEL1 raw slot");
constexpr uint32_t P_BYTES = 64 * 128;
constexpr uint32_t QROPE_BYTES = 64 * 128;          // Q's RoPE part of this CTA's 64 heads: one 128B-swizzled [64 x 64] panel
// tensor memory: O | Q (NoPE half of the lane: 256 dims, two per column) | two S buffers
constexpr uint32_t TM_O = 0, TM_Q = 256, TM_S = 384, TM_COLS = 512;
// Registers per thread after the warpgroups have re-divided the register file.  The pool is what the launch gave the
// CTA (80 per thread with 768 threads, 96 with 640: the most they can have), not the SM's whole file: an increase
// beyond it never returns.
constexpr int REGS_SOFTMAX = 128, REGS_GATHER = 40;
constexpr int regs_launch(bool raw) { return raw ? 80 : 96; }
constexpr int regs_producer(bool raw) { return raw ? 64 : 80; }
constexpr int regs_issuer(bool raw) { return raw ? 56 : 64; }
static_assert(NSW * REGS_SOFTMAX + NPW * regs_producer(true) + 4 * regs_issuer(true) + NGW * REGS_GATHER <= (NSW + NPW + 4 + NGW) * regs_launch(true) &&
              NSW * REGS_SOFTMAX + NPW * regs_producer(false) + 4 * regs_issuer(false) <= (NSW + NPW + 4) * regs_launch(false), "register pool");
static_assert(NSW % 4 == 0 && NPW % 4 == 0 && NGW % 4 == 0, "roles fill whole warpgroups");
constexpr float RESCALE_THRESHOLD = 6.f;   // log2 units the block maximum may exceed the reference maximum
constexpr int RING = 8;                    // slots of the index and validity-mask rings
constexpr int IDX_LOOKAHEAD = 6;           // prefill: blocks the index prefetch runs ahead of the gathers

// shared-memory map (offsets from a 1024-byte aligned base)
enum Bar { KV_FULL = 0, KV_EMPTY = KV_FULL + MAX_STAGES, RAW_FULL = KV_EMPTY + MAX_STAGES /* [NGW][NRAW] */, RAW_EMPTY = RAW_FULL + NGW * NRAW /* [NGW][NRAW] */,
           S_FULL = RAW_EMPTY + NGW * NRAW /* [2 teams] */, S_EMPTY = S_FULL + 2 /* [2 teams] */, P_FULL = S_EMPTY + 2 /* [2 teams] */,
           PV_DONE = P_FULL + 2 /* [2 teams] */, DEC = PV_DONE + 2 /* [2 teams] */, Q_FULL = DEC + 2, QL_FULL /* [2 item parities] */, O_FREE = QL_FULL + 2, NUM_BARS };
constexpr uint32_t SM_BAR = 0;
constexpr uint32_t SM_TMEM = SM_BAR + NUM_BARS * 8;
constexpr uint32_t SM_ABORT = SM_TMEM + 4;
constexpr uint32_t SM_LEAVE = SM_ABORT + 4;                 // softmax warps that have left because of an abort
constexpr uint32_t SM_MASK = 512;                           // uint8 [RING][8]: validity bits of the block's tokens 8w .. 8w+7
constexpr uint32_t SM_XFLAG = SM_MASK + RING * 8;           // uint8 [NGW][RING] (decode over two caches): the block's rows live in the extra cache
constexpr uint32_t SM_MAX = 1024;                           // float [2 teams][2 halves][64]: block maxima of a thread's 32 tokens
constexpr uint32_t SM_MREF = SM_MAX + 1024;                 // float [2 teams][64]: reference maximum after the team's latest block
constexpr uint32_t SM_MTRUE = SM_MREF + 512;                // float [2 teams][64]: largest logit of the team's blocks, at the end of a query
constexpr uint32_t SM_SUM = SM_MAX + 2048;                  // float [4][64]: row sums at the end of a query
constexpr uint32_t SM_IDX = SM_SUM + 1024;                  // int32 [NPW producer warps][RING][PROWS] / [NGW gather warps][RING][GROWS]
constexpr uint32_t SM_P = 6144;                             // two P buffers (one per team), 1024-byte aligned
constexpr uint32_t XCHG_BYTES = 2 * 2 * 32 * 64;           // one of the two halves of the partial-sum exchange (the other half travels through the team's P buffer)
constexpr uint32_t SM_XCHG = SM_P + 2 * P_BYTES;            // float [2 head ranges][2 receiving halves][32 heads][16], chunk-swizzled; also a Q tile
constexpr uint32_t SM_QROPE = SM_XCHG + XCHG_BYTES;         // Q's RoPE panel (A operand of the RoPE k-steps)
constexpr uint32_t SM_STAGE = SM_QROPE + QROPE_BYTES;       // stages, then (decode) the raw ring
constexpr uint32_t SM_RAW = SM_STAGE + NSTAGE_DECODE * STAGE_BYTES;
static_assert(XCHG_BYTES == P_BYTES && SM_LEAVE + 4 <= SM_MASK && SM_XFLAG + NPW * RING <= SM_MAX && SM_MTRUE + 512 <= SM_SUM && SM_IDX + NPW * RING * PROWS * 4 <= SM_P && SM_P % 1024 == 0 &&
              SM_QROPE % 1024 == 0 && SM_STAGE % 1024 == 0 && STAGE_BYTES % 1024 == 0 && SM_RAW % 1024 == 0 && RAW_BYTES % 1024 == 0 && SM_BAR + 8 * NUM_BARS + 12 <= SM_MASK,
              "shared memory map");
constexpr uint32_t SM_XCHG2 = SM_STAGE + NSTAGE_PREFILL * STAGE_BYTES;   // prefill: the second half of the exchange has a buffer of its own
constexpr uint32_t SMEM_USED_PREFILL = SM_XCHG2 + XCHG_BYTES;
constexpr uint32_t SMEM_USED_DECODE = SM_RAW + NRAW * RAW_BYTES;
constexpr uint32_t SMEM_BYTES = (SMEM_USED_PREFILL > SMEM_USED_DECODE ? SMEM_USED_PREFILL : SMEM_USED_DECODE) + 1024;
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget exceeded");

struct Params {
  CUtensorMap map_nope, map_rope;   // decode: byte views of the pool (256-byte NoPE box, 64-byte RoPE box); prefill: bf16 views of kv (64 / 32 dims)
                                    // MODEL1 decode: 576-byte-pitch views with boxes of 256 (map_nope), 192 (map_rope) and 128 bytes (map_scale)
  CUtensorMap map_scale;            // decode: byte view of the pool with a 16-byte box (the scale field of a row)
  CUtensorMap map_nope2, map_rope2, map_scale2;   // the same for the extra cache
  CUtensorMap map_q;               // q as (576, h_q, s_q, b) / (576, h_q, queries, 1): boxes of 64 heads x 64 dims (128B swizzle)
  CUtensorMap map_q_rope;          // the same view with boxes of 64 heads x 32 dims (64B swizzle)
  int q_tma;                     // the map above is valid; else Q is read with plain loads
  CUtensorMap map_out;             // out as (512, h_q, s_q, b) / (512, h_q, queries, 1) bf16: boxes of 32 heads x 32 dims (64B swizzle)
  CUtensorMap map_acc;             // decode: o_accum as (512, h_q, rows / h_q, 1) fp32: boxes of 32 heads x 16 dims (64B swizzle)
  int out_tma;                   // the two maps above are valid; else the epilogue stores with plain stores
  // decode with a second cache (extra_k_cache): its maps, geometry and index list; has_extra = 0 otherwise
  int has_extra, page2, rows_per_block2, extra_topk;
  int64_t total_rows2, kv_stride_block2;
  const uint8_t* kv_rows2;
  const int* indices2;
  int64_t idx2_stride0, idx2_stride1;
  const int* extra_topk_length;
  int mode;                      // 0 decode, 1 prefill
  int h_q, topk;
  int d_qk;                      // values per q / kv row: 576, or 512 (prefill only; the missing RoPE part reads as zero)
  float scale_log2;
  const __nv_bfloat16* q;
  int64_t q_stride0, q_stride1, q_stride_h;   // decode: batch, s_q; prefill: query, unused
  const int* indices;
  int64_t idx_stride0, idx_stride1;
  const int* topk_length;
  const float* attn_sink;
  // decode
  const uint8_t* kv_rows;
  int64_t kv_stride_block;
  int page, layout;
  int rows_per_block;            // decode: rows of the 656-byte-pitch view per cache block = block stride / 656
  int64_t total_rows;
  const SchedRecord* sched;
  const int* block_table;        // dense decode: [b][block_table_stride] cache blocks of each request, in order
  int64_t block_table_stride;
  int causal;                    // dense decode: row sq of a request's s_q rows sees its first len - (s_q - 1 - sq) tokens
  int dense_blocks;              // dense decode: blocks in the cache (block-table entries outside [0, dense_blocks) are invalid slots)
  const int* num_splits;
  int b, s_q;
  __nv_bfloat16* out;
  int64_t o_stride0, o_stride1, o_stride_h;
  float* lse;
  int64_t lse_stride0, lse_stride1;
  float* o_accum;
  float* lse_accum;
  // prefill
  const __nv_bfloat16* kv_bf16;
  int64_t kv_stride_s;
  int s_kv, n_queries;
  float* max_logits;
  int* status;
};
// Params with the mode as a compile-time constant: `p.mode` in the device code below resolves to it, so each
// instantiation of the kernel carries the code of one mode only.
// VARIANT (decode): 0 = one cache of 656-byte rows, 1 = two such caches, 2 = one cache of MODEL1 blocks (d_qk = 512),
// 3 = dense decode: a bf16 cache of which every request attends all its tokens, found through its block table,
// 4 = two caches of MODEL1 blocks
template <int MODE, int VARIANT>
struct ParamsT : Params {
  static constexpr int mode = MODE;
  static constexpr int has_extra = VARIANT == 1 || VARIANT == 4;   // decode over two caches; a compile-time constant like the mode
  static constexpr int m1 = VARIANT == 2 || VARIANT == 4;          // MODEL1 rows: 448 e4m3 + 64 bf16, V = all 512 values
  static constexpr int dense = VARIANT == 3;         // bf16 rows gathered straight into the stages, as in prefill
  static constexpr int raw = raw_ring(MODE, VARIANT);      // rows pass through the raw ring and are dequantised into fp16 stages:
                                                           // K, V, Q (NoPE) and P are then fp16, else bf16
};

struct Item {
  const __nv_bfloat16* q;   // head 0 of this query
  const int* idx;
  int tok_lo, tok_hi, limit;   // token range of this piece in the request's token list; main slots >= limit are masked
  const int* idx2;             // extra index list (token list positions main_end .. limit2-1), or unused
  int main_end, limit2;
  int split;                // decode: write fp32 partials to the accumulators
  int64_t row;              // split: accumulator row of head 0; prefill: query index
  int req, sq;
};

// i-th work item of this pair; false when the list is exhausted.
template <class P>
__device__ __forceinline__ bool get_item(const P& p, const SchedRecord& rec, int i, Item& it) {
  if (p.mode == 0) {
    const int req = rec.begin_req + i;
    if (rec.begin_req >= p.b || req > rec.end_req) return false;
    const int sq = blockIdx.y;
    const int blk_lo = req == rec.begin_req ? rec.begin_block : 0;
    int lim = p.topk_length ? __ldg(p.topk_length + req) : p.topk;
    if (p.dense && p.causal) lim -= p.s_q - 1 - sq;          // the request's last s_q tokens are the queries themselves
    it.limit = lim < p.topk ? (lim < 0 ? 0 : lim) : p.topk;
    int total = p.topk;
    it.main_end = 0x7fffffff; it.limit2 = 0; it.idx2 = nullptr;
    if (p.has_extra) {           // the extra slots follow the main ones from the next block boundary, as the scheduler counts them
      const int s_main = lim <= 0 ? 1 : lim;
      int e = p.extra_topk_length ? __ldg(p.extra_topk_length + req) : p.extra_topk;
      e = e < 0 ? 0 : (e < p.extra_topk ? e : p.extra_topk);
      it.main_end = (s_main + T - 1) / T * T;
      it.limit2 = total = it.main_end + e;
      it.idx2 = p.indices2 + req * p.idx2_stride0 + blockIdx.y * p.idx2_stride1;
    }
    const int64_t hi = req == rec.end_req ? (int64_t)rec.end_block * T : (int64_t)total;
    it.tok_lo = blk_lo * T;
    it.tok_hi = (int)(hi < total ? hi : total);
    if (it.tok_hi <= it.tok_lo) it.tok_hi = it.tok_lo + 1;   // a scheduled piece always runs one (masked) block
    it.split = req == rec.begin_req ? rec.first_split : (req == rec.end_req ? rec.last_split : 0);
    it.q = p.q + req * p.q_stride0 + sq * p.q_stride1;
    it.idx = p.indices + req * p.idx_stride0 + sq * p.idx_stride1;
    it.req = req; it.sq = sq;
    it.row = 0;
    if (it.split) {
      const int slot = __ldg(p.num_splits + req) + (req == rec.begin_req ? rec.begin_split : 0);
      it.row = ((int64_t)slot * p.s_q + sq) * p.h_q;
    }
    return true;
  }
  const int nclusters = gridDim.x >> 1;
  const int qi = (int)(blockIdx.x >> 1) + i * nclusters;
  if (qi >= p.n_queries) return false;
  it.tok_lo = 0;
  int lim = p.topk_length ? __ldg(p.topk_length + qi) : p.topk;
  lim = lim < 0 ? 0 : (lim < p.topk ? lim : p.topk);
  it.limit = lim;
  it.tok_hi = lim > 0 ? lim : 1;
  it.main_end = 0x7fffffff; it.limit2 = 0; it.idx2 = nullptr;
  it.split = 0;
  it.q = p.q + qi * p.q_stride0;
  it.idx = p.indices + qi * p.idx_stride0;
  it.req = qi; it.sq = 0; it.row = qi;
  return true;
}

__device__ __forceinline__ int num_blocks(const Item& it) { return (it.tok_hi - it.tok_lo + T - 1) / T; }

template <int N> __device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

// ---- abort plumbing ----------------------------------------------------------------------------
struct Ctx {
  uint32_t base;            // shared::cta address of the aligned smem base
  volatile int* abort_flag; // generic pointer to SM_ABORT
  uint32_t peer;            // rank of the other CTA
  int* status;
};
__device__ __noinline__ void raise_abort(const Ctx& c, int code) {
  *c.abort_flag = code;
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(map_to_cta(c.base + SM_ABORT, c.peer)), "r"(code) : "memory");
  if (c.status) atomicCAS(c.status, 0, code);
}
__device__ __forceinline__ uint32_t bar_addr(const Ctx& c, int bar) { return c.base + SM_BAR + 8u * bar; }
// Bounded wait; false means the kernel is aborting.
__device__ __forceinline__ bool wait(const Ctx& c, int bar, uint32_t parity, int code) {
  if (mbar_wait_abortable(bar_addr(c, bar), parity & 1u, c.abort_flag)) return true;
  if (*c.abort_flag == 0) raise_abort(c, code);
  return false;
}
// Arrive on barrier `bar` of CTA 0 (the MMA issuers live there).
__device__ __forceinline__ void arrive_leader(const Ctx& c, int bar) {
  if (c.peer == 1u) mbar_arrive(bar_addr(c, bar));                 // this CTA is the leader
  else mbar_arrive_cluster(map_to_cta(bar_addr(c, bar), 0));
}

// ---- shared-memory helpers ---------------------------------------------------------------------------
__device__ __forceinline__ float lds_f32(uint32_t a) { float v; asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a)); return v; }
__device__ __forceinline__ void sts_u32(uint32_t a, uint32_t v) { asm volatile("st.shared.u32 [%0], %1;" ::"r"(a), "r"(v) : "memory"); }
__device__ __forceinline__ void sts_f32(uint32_t a, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory"); }
__device__ __forceinline__ uint32_t lds_u32(uint32_t a) { uint32_t v; asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a)); return v; }
__device__ __forceinline__ uint4 lds_16(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t stage_addr(const Ctx& c, int s) { return c.base + SM_STAGE + (uint32_t)s * STAGE_BYTES; }
template <class P>
__device__ __forceinline__ int num_stages(const P& p) { return p.raw ? NSTAGE_DECODE : NSTAGE_PREFILL; }

// Enumerates the blocks of all work items in order (registers only).
struct BlockCursor {
  Item it;
  int item, n;
  bool live;
  template <class P>
  __device__ BlockCursor(const P& p, const SchedRecord& rec) { item = 0; n = 0; live = get_item(p, rec, 0, it); }
  template <class P>
  __device__ __forceinline__ void advance(const P& p, const SchedRecord& rec) {
    if (++n >= num_blocks(it)) { n = 0; ++item; live = get_item(p, rec, item, it); }
  }
};

// ---- TMA gathers ---------------------------------------------------------------------------------------
// Four rows of a 2-D tensor map into four consecutive rows of this CTA's shared memory (destination 128-byte aligned),
// completion on a local mbarrier; rows outside the tensor are zero-filled.
__device__ __forceinline__ void tma_gather4(uint32_t dst, const CUtensorMap* map, int col, int4 rows, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes.cta_group::1 [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
      ::"r"(dst), "l"(map), "r"(col), "r"(rows.x), "r"(rows.y), "r"(rows.z), "r"(rows.w), "r"(bar) : "memory");
}
// Four rows of a 2-D tensor map into four consecutive rows of shared memory (destination 128-byte aligned);
// rows outside the tensor are zero-filled.  `col` times the element size must be a multiple of 16 bytes.
// The completion is signalled on a barrier given by a shared::cluster address, which may
// belong to the other CTA of the pair (cta_group::2); the destination is this CTA's own shared memory.
__device__ __forceinline__ void tma_gather4_pair(uint32_t dst, const CUtensorMap* map, int col, int4 rows, uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes.cta_group::2 [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
      ::"r"(dst), "l"(map), "r"(col), "r"(rows.x), "r"(rows.y), "r"(rows.z), "r"(rows.w), "r"(cluster_bar) : "memory");
}
// One arrival plus `bytes` of expected transactions on a barrier given by a shared::cluster address.
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t cluster_bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// 4-D tile load into this CTA's shared memory, completion on a local mbarrier.
__device__ __forceinline__ void tma_tile_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar) : "memory");
}

// 4-D tile store from this CTA's shared memory (bulk async group of the issuing thread).  No coordinate is negative.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3, %4}], [%5];"
               ::"l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(src) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the issuing thread's bulk stores have read their shared-memory source / have completed
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---- Q travels through the stage ring -------------------------------------------------------------------
// The stages are used in a fixed order of ring positions.  The two positions before the first block of a work item
// hold that item's Q: position k = feature half k of this CTA's 64 heads, laid out exactly like a stage of KV rows (four
// 128B-swizzled NoPE tiles of 64 dims and one 64B-swizzled RoPE tile of 32 dims, the heads in place of the tokens).  So
// Q is fetched by the warps that fill the stages, as far ahead as the KV rows, and lies ready when the softmax warps
// move it into tensor memory at the end of the item before.  Block n of the i-th item of a pair sits at ring position
// (blocks of the items before) + n + 2 (i + 1).
// Called by all lanes of a stage-filling warp (`pwarp` of NPW) at the start of an item: warps 0-3 fetch NoPE tile
// `pwarp`, warp 4 the RoPE tile, of both positions; the bytes are counted on this CTA's QL_FULL barrier of the item's
// parity (items alternate between two barriers: the ring may hold the Q of two short items at once, but never of three),
// and every warp arrives on the leader's stage barrier so that its phase stays in step with the stage's uses.  `item`
// is the item's number in the pair's list, (c2, c3) its outer coordinates in q.  Returns false when the kernel is aborting.
template <class P>
__device__ __forceinline__ bool fill_q_positions(const P& p, const Ctx& c, uint32_t rank, int pwarp, int lane, int item, int c2, int c3, uint32_t& pos) {
  const int nst = num_stages(p);
  const int head0 = blockIdx.z * 128 + (int)rank * 64;
#pragma unroll 1
  for (int k = 0; k < 2; ++k, ++pos) {
    const int st = pos % nst;
    const uint32_t use = pos / nst;
    const bool ok = use == 0 || wait(c, KV_EMPTY + st, use - 1, 16);
    if (!__all_sync(0xffffffffu, ok)) return false;
    if (lane == 0) {
      if (pwarp < 5) {
        const uint32_t bar = bar_addr(c, QL_FULL + (item & 1)), dst = c.base + SM_STAGE + (uint32_t)st * STAGE_BYTES;
        if (!p.q_tma) mbar_arrive(bar);                 // Q is read with plain loads: nothing to fetch
        else if (pwarp < 4) {
          mbar_expect_tx(bar, PANEL);
          tma_tile_4d(dst + pwarp * PANEL, &p.map_q, 256 * k + 64 * pwarp, head0, c2, c3, bar);
        } else {
          mbar_expect_tx(bar, T * 64);
          tma_tile_4d(dst + ROPE_PANEL, &p.map_q_rope, 512 + 32 * k, head0, c2, c3, bar);
        }
      }
      arrive_leader(c, KV_FULL + st);
    }
  }
  return true;
}

// ---- FP8 dequantisation (decode) --------------------------------------------------------------------------
// Decode stages the NoPE half in fp16, not bf16: e4m3 -> f16 is one exact conversion per pair and the scale
// is one packed multiply, four times fewer instructions than going through fp32 to bf16.  fp8 * 2^k is exact
// in fp16 just as in bf16 while |value| <= 57344 (scales are clamped to 2^7) and above fp16's sub-normal
// range; the QK^T (NoPE k-steps) and PV products of a decode launch therefore run as fp16 x fp16 MMAs with Q
// and P converted to fp16, and only the RoPE k-steps stay bf16 x bf16.
__device__ __forceinline__ uint32_t cvt_e4m3x2_f16x2(uint32_t two_bytes) {
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)two_bytes, __NV_E4M3);
  return (uint32_t)h.x | ((uint32_t)h.y << 16);
}
__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
// fp32 scale -> packed half2 scale, clamped to [0, 2^7]: e4m3 times a larger scale can leave fp16's range
constexpr float MAX_STAGED_SCALE = 128.f;
__device__ __forceinline__ uint32_t scale_to_half2(float scale) {
  const __half h = __float2half_rn(fminf(scale, MAX_STAGED_SCALE));
  const uint32_t u = (uint32_t)__half_as_ushort(h);
  return u | (u << 16);
}
__device__ __forceinline__ void dequant_chunk_f16(const uint4& raw, uint32_t scale_h2, uint4& out_lo, uint4& out_hi) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    o[2 * i] = hmul2(cvt_e4m3x2_f16x2(w[i] & 0xffffu), scale_h2);
    o[2 * i + 1] = hmul2(cvt_e4m3x2_f16x2(w[i] >> 16), scale_h2);
  }
  out_lo = make_uint4(o[0], o[1], o[2], o[3]);
  out_hi = make_uint4(o[4], o[5], o[6], o[7]);
}

// running maximum of |x| over packed bf16 pairs
__device__ __forceinline__ uint32_t absmax_bf16x2(uint32_t acc, uint32_t v) {
  uint32_t r;
  asm("{\n\t.reg .b32 t;\n\tabs.bf16x2 t, %2;\n\tmax.bf16x2 %0, %1, t;\n\t}" : "=r"(r) : "r"(acc), "r"(v));
  return r;
}
// whether a packed pair of non-negative bf16 holds a value beyond fp16's largest (65504; the next bf16 is 65536 = 0x4780)
__device__ __forceinline__ bool beyond_f16(uint32_t absmax) { return (((absmax & 0x7fff7fffu) + 0x38803880u) & 0x80008000u) != 0u; }
// bf16 pair -> fp16 pair (values beyond fp16's range saturate to +-65504)
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t v) {
  uint32_t r;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(__uint_as_float(v & 0xffff0000u)), "f"(__uint_as_float(v << 16)));
  return r;
}
// ---- prefill: producer warps --------------------------------------------------------------------------------
// Producer warp w (of NPW) owns tokens [PROWS*w, PROWS*(w+1)) of every block.  Its loop is a chain of dependent
// shared-memory reads, shuffles and waits around ten gathers, and the eight warps together are the slowest link of the
// prefill pipeline; so a warp takes two blocks per turn and pays for everything but the gathers once per pair:
//   * lanes 0-15 prefetch the indices of the pair three turns ahead into the warp's ring (4-byte cp.async), lanes 0-7
//     those of block 2i and lanes 8-15 those of block 2i+1, each lane with the block cursor of its own block;
//   * lane = 10 block + 5 group + piece (20 lanes) reads the four indices of its group and, once the block's stage is
//     free, issues one TMA gather of four bf16 rows (piece = NoPE panel 0-3 / RoPE panel) straight into the swizzled
//     stage.  The warp's arrival and the gathers' bytes go to the leader CTA's stage barrier, so nobody waits for the
//     landing in between and the gathers run as far ahead of the MMAs as stages are free.
template <class P>
__device__ void producer_role(const P& p, const SchedRecord& rec, const Ctx& c, uint32_t rank) {
  const int ptid = threadIdx.x - 32 * NSW, pwarp = ptid >> 5, lane = ptid & 31;
  constexpr int nst = NSTAGE_PREFILL;
  const int range = p.s_kv;
  const uint32_t ring = c.base + SM_IDX + (uint32_t)pwarp * (RING * PROWS * 4);
  static_assert(PROWS == 8 && RING % 2 == 0, "two four-row groups per producer warp and block");
  const int fsub = (lane >> 3) & 1, frow = lane & 7;  // feeding lanes 0-15: block of the pair, row
  BlockCursor feed(p, rec), gat(p, rec);
  if (fsub && feed.live) feed.advance(p, rec);        // lanes 8-15 walk the odd blocks

  // Dense decode has no index lists: token t of a request is row block_table[request][t / page] * page + t % page of the
  // cache.  The ring then carries the cache block of each token, and the first token position of a block travels from
  // the feeding lanes to the issuing lanes through a three-deep queue in registers (base0 = the pair being gathered).
  int base0 = 0, base1 = 0, base2 = 0;
  auto feed_pair = [&](uint32_t j) {          // indices of blocks 2j, 2j+1 -> ring slots (2j + fsub) % RING; one cp.async group
    int base = 0;
    if (lane < 2 * PROWS && feed.live) {
      base = feed.it.tok_lo + feed.n * T;
      const int pos = base + PROWS * pwarp + frow;
      const uint32_t dst = ring + (((2 * j + fsub) % RING) * PROWS + frow) * 4;
      const int* src = p.dense ? p.block_table + feed.it.req * p.block_table_stride + pos / p.page : feed.it.idx + pos;
      if (pos < feed.it.tok_hi && pos < feed.it.limit)
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
      else
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(dst), "r"(0xffffffffu) : "memory");
      feed.advance(p, rec);
      if (feed.live) feed.advance(p, rec);
    }
    cp_async_commit();
    if (p.dense) { base0 = base1; base1 = base2; base2 = base; }
  };

#pragma unroll 1
  for (int k = 0; k < 3; ++k) feed_pair(k);
  const int sub = lane / 10, rem = lane - 10 * sub, q = rem / 5, kind = rem - 5 * q;   // issuing lanes 0-19
  const bool issuer = lane < 20;
  uint32_t pos = 0;                                   // ring position
  for (uint32_t i = 0; gat.live; ++i) {
    // pairs 0 .. i+2 are committed; with at most two groups pending, pair i has landed
    cp_async_wait<2>();
    __syncwarp();
    uint32_t bits = 0;
    int id[4] = {-1, -1, -1, -1};
    if (issuer) {
      const uint4 v = lds_16(ring + (((2 * i + sub) % RING) * PROWS + 4 * q) * 4);
      id[0] = (int)v.x; id[1] = (int)v.y; id[2] = (int)v.z; id[3] = (int)v.w;
    }
    if (p.dense) {                  // cache block -> cache row (all lanes take part in the shuffle)
      const int base = __shfl_sync(0xffffffffu, base0, 8 * sub) + PROWS * pwarp + 4 * q;
#pragma unroll
      for (int k = 0; k < 4; ++k)
        id[k] = id[k] >= 0 && id[k] < p.dense_blocks ? id[k] * p.page + (base + k) % p.page : -1;   // a block the cache does not have: invalid slot
    }
    if (issuer) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (id[k] < 0 || id[k] >= range) { id[k] = -1; continue; }      // the TMA unit zero-fills row -1
        if (kind == 0) bits |= 1u << (4 * q + k);                       // one lane per group reports validity
      }
    }
    bits |= __shfl_xor_sync(0xffffffffu, bits, 5);                     // lanes 0 / 10 hold the two groups of block 0 / 1
#pragma unroll 1
    for (int s = 0; s < 2 && gat.live; ++s, ++pos, gat.advance(p, rec)) {
      const uint32_t g = 2 * i + s;
      if (gat.n == 0 && !fill_q_positions(p, c, rank, pwarp, lane, gat.item, p.mode == 0 ? gat.it.sq : gat.it.req, p.mode == 0 ? gat.it.req : 0, pos)) return;
      const int st = pos % nst;
      const uint32_t use = pos / nst;
      const bool ok = use == 0 || wait(c, KV_EMPTY + st, use - 1, 12);
      if (!__all_sync(0xffffffffu, ok)) return;
      const uint32_t dst = stage_addr(c, st);
      const uint32_t bar = map_to_cta(bar_addr(c, KV_FULL + st), 0);      // shared::cluster address of the leader's stage barrier
      if (lane == 10 * s) {
        asm volatile("st.shared.u8 [%0], %1;" ::"r"(c.base + SM_MASK + 8u * (g % RING) + pwarp), "r"(bits) : "memory");
        mbar_expect_tx_cluster(bar, STAGE_TX_BYTES / NPW);               // after the mask store
      }
      __syncwarp();
      if (issuer && sub == s) {
        const uint32_t r0 = (uint32_t)PROWS * pwarp + 4u * q;             // first of the four stage rows
        const uint32_t d = kind < 4 ? dst + kind * PANEL + r0 * 128u : dst + ROPE_PANEL + r0 * 64u;
        const CUtensorMap* map = kind < 4 ? &p.map_nope : &p.map_rope;
        const int col = kind < 4 ? 256 * (int)rank + 64 * kind : 512 + 32 * (int)rank;
        tma_gather4_pair(map_to_cta(d, rank), map, col, make_int4(id[0], id[1], id[2], id[3]), bar);
      }
    }
    feed_pair(i + 3);
  }
  cp_async_wait<0>();
}

// ---- decode: gather warps and converter warps ---------------------------------------------------------
// Gather warp w (of NGW) brings rows [GROWS*w, GROWS*(w+1)) of every block into the raw ring:
//   * lanes 0-15 prefetch the rows' cache indices into the warp's ring (4-byte cp.async, IDX_LOOKAHEAD blocks ahead);
//   * once the raw slot is free, lane = 4 piece + group (12 lanes) issues one TMA gather of four rows: piece 0 = this
//     CTA's NoPE half (256 bytes per row), 1 = this CTA's RoPE half (64 bytes), 2 = the scale field (16 bytes).  An
//     invalid slot gets row -1, which the TMA unit zero-fills, so it contributes exact zeros even when unused rows are
//     NaN-poisoned.
// A gather costs its issuing warp some 70 cycles whatever the lane, and warps issue in parallel: hence four warps.
// The eight converter warps dequantise eight rows each from the raw ring into the stage and tell the leader CTA.
template <class P>
__device__ void gather_role(const P& p, const SchedRecord& rec, const Ctx& c, uint32_t rank, int gw) {
  const int lane = threadIdx.x & 31;
  const uint32_t ring = c.base + SM_IDX + (uint32_t)gw * (RING * GROWS * 4);
  const uint32_t flags = c.base + SM_XFLAG + (uint32_t)gw * RING;     // per block: its rows live in the extra cache
  BlockCursor feed(p, rec);
  uint32_t total_blocks = 0;
  {
    Item it;
    for (int i = 0; get_item(p, rec, i, it); ++i) total_blocks += (uint32_t)num_blocks(it);
  }
  auto feed_block = [&](uint32_t blk) {       // cache indices of block blk -> ring slot blk % RING; one cp.async group
    if (feed.live) {
      // a block lies entirely in the main or in the extra part of the token list (the boundary is a block multiple)
      if (p.has_extra && lane == 0)
        asm volatile("st.shared.u8 [%0], %1;" ::"r"(flags + blk % RING), "r"(feed.it.tok_lo + feed.n * T >= feed.it.main_end ? 1u : 0u) : "memory");
      if (lane < GROWS) {
        const int pos = feed.it.tok_lo + feed.n * T + GROWS * gw + lane;
        const uint32_t dst = ring + ((blk % RING) * GROWS + lane) * 4;
        const int* src = nullptr;
        if (pos < feed.it.tok_hi) {
          if (pos < feed.it.main_end) { if (pos < feed.it.limit) src = feed.it.idx + pos; }
          else if (pos < feed.it.limit2) src = feed.it.idx2 + (pos - feed.it.main_end);
        }
        if (src) asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
        else asm volatile("st.shared.u32 [%0], %1;" ::"r"(dst), "r"(0xffffffffu) : "memory");
      }
      feed.advance(p, rec);
    }
    cp_async_commit();
  };
#pragma unroll 1
  for (int k = 0; k < IDX_LOOKAHEAD; ++k) feed_block(k);
  const int grp = lane & 3, piece = lane >> 2;
  // MODEL1: row lane % 16 of block blk as a row number of the pool's 576-byte-pitch view (-1: invalid slot), and the
  // row's eight scale bytes, which sit behind the block's data rows: read with a plain load one block ahead of the
  // gathers and stored into the raw slot by this warp (zero for an invalid slot: its data bytes are zero-filled)
  auto m1_row = [&](uint32_t blk, uint2& scales) -> int {
    scales = make_uint2(0u, 0u);
    if (blk >= total_blocks) return -1;
    const int id = (int)lds_u32(ring + ((blk % RING) * GROWS + (lane & 15)) * 4);
    bool extra = false;
    if (p.has_extra) { uint32_t f; asm volatile("ld.shared.u8 %0, [%1];" : "=r"(f) : "r"(flags + blk % RING)); extra = f != 0; }
    if (id < 0 || id >= (extra ? p.total_rows2 : p.total_rows)) return -1;
    const int page = extra ? p.page2 : p.page;
    const int b = id / page, off = id - b * page;
    const uint8_t* pool = extra ? p.kv_rows2 + (int64_t)b * p.kv_stride_block2 : p.kv_rows + (int64_t)b * p.kv_stride_block;
    scales = ldg_nc_8(pool + (int64_t)page * M1_DATA_BYTES + off * 8);
    return b * (extra ? p.rows_per_block2 : p.rows_per_block) + off;
  };
  uint2 m1_scales = make_uint2(0u, 0u);
  int m1_vrow = -1;
  if (p.m1) {
    cp_async_wait<IDX_LOOKAHEAD - 1>();
    __syncwarp();
    m1_vrow = m1_row(0, m1_scales);
  }
  for (uint32_t g = 0; g < total_blocks; ++g) {
    // groups 0 .. g+IDX_LOOKAHEAD-1 are committed; with at most IDX_LOOKAHEAD-1 pending, group g has landed (MODEL1
    // looks one block further)
    if (p.m1) cp_async_wait<IDX_LOOKAHEAD - 2>(); else cp_async_wait<IDX_LOOKAHEAD - 1>();
    __syncwarp();
    bool extra = false;
    if (p.has_extra) { uint32_t f; asm volatile("ld.shared.u8 %0, [%1];" : "=r"(f) : "r"(flags + g % RING)); extra = f != 0; }
    int vrow = -1;
    uint2 m1_scales_next = make_uint2(0u, 0u);
    int m1_vrow_next = -1;
    if (p.m1) {
      vrow = m1_vrow;
      m1_vrow_next = m1_row(g + 1, m1_scales_next);
    } else {
      const int64_t total = extra ? p.total_rows2 : p.total_rows;
      const int page = extra ? p.page2 : p.page, rpb = extra ? p.rows_per_block2 : p.rows_per_block;
      // row lane % 16 of the warp as a row number of the pool's 656-byte-pitch view (a cache block may be padded by whole rows)
      const int id = (int)lds_u32(ring + ((g % RING) * GROWS + (lane & 15)) * 4);
      if (id >= 0 && id < total) {
        if (rpb == page) vrow = id;
        else { const int b = id / page; vrow = b * rpb + (id - b * page); }
      }
    }
    const uint32_t bits = __ballot_sync(0xffffffffu, vrow >= 0) & 0xffffu;
    int4 rows;
    rows.x = __shfl_sync(0xffffffffu, vrow, 4 * grp);
    rows.y = __shfl_sync(0xffffffffu, vrow, 4 * grp + 1);
    rows.z = __shfl_sync(0xffffffffu, vrow, 4 * grp + 2);
    rows.w = __shfl_sync(0xffffffffu, vrow, 4 * grp + 3);
    const int slot = g % NRAW;
    const uint32_t use = g / NRAW;
    const bool ok = use == 0 || wait(c, RAW_EMPTY + gw * NRAW + slot, use - 1, 12);
    if (!__all_sync(0xffffffffu, ok)) return;
    const uint32_t bar = bar_addr(c, RAW_FULL + gw * NRAW + slot);
    const uint32_t dst = c.base + SM_RAW + (uint32_t)slot * RAW_BYTES;
    const uint32_t q = (uint32_t)(4 * gw + grp);                   // group of four rows within the block
    if (p.m1) {
      if (lane < GROWS)
        asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(dst + M1_RAW_SCALE + (uint32_t)(GROWS * gw + lane) * 8u), "r"(m1_scales.x), "r"(m1_scales.y) : "memory");
      if (lane == 0) asm volatile("st.shared.u16 [%0], %1;" ::"r"(c.base + SM_MASK + 8u * (g % RING) + 2u * gw), "r"(bits) : "memory");
      __syncwarp();                   // the stores above happen before the arrival below
      if (lane == 0) mbar_expect_tx(bar, GROWS * (rank == 0 ? 256u : 320u));
      if (rank == 0) {
        if (piece == 0) tma_gather4(dst + q * 1024u, extra ? &p.map_nope2 : &p.map_nope, 0, rows, bar);
      } else {
        if (piece == 0) tma_gather4(dst + q * 768u, extra ? &p.map_rope2 : &p.map_rope, 256, rows, bar);
        else if (piece == 1) tma_gather4(dst + M1_RAW_ROPE + q * 512u, extra ? &p.map_scale2 : &p.map_scale, M1_D_NOPE, rows, bar);
      }
      m1_vrow = m1_vrow_next;
      m1_scales = m1_scales_next;
      feed_block(g + IDX_LOOKAHEAD);
      continue;
    }
    if (lane == 0) {
      asm volatile("st.shared.u16 [%0], %1;" ::"r"(c.base + SM_MASK + 8u * (g % RING) + 2u * gw), "r"(bits) : "memory");
      mbar_expect_tx(bar, RAW_TX_BYTES);
    }
    __syncwarp();
    if (piece == 0) tma_gather4(dst + RAW_NOPE + q * 1024u, extra ? &p.map_nope2 : &p.map_nope, 256 * (int)rank, rows, bar);
    else if (piece == 1) tma_gather4(dst + RAW_ROPE + q * ROPE_GROUP, extra ? &p.map_rope2 : &p.map_rope, ROPE_OFF + 64 * (int)rank, rows, bar);
    else if (piece == 2) tma_gather4(dst + RAW_SCALE + q * SCALE_GROUP, extra ? &p.map_scale2 : &p.map_scale, SCALE_OFF, rows, bar);
    feed_block(g + IDX_LOOKAHEAD);
  }
  cp_async_wait<0>();
}

template <class P>
__device__ void convert_role(const P& p, const SchedRecord& rec, const Ctx& c, uint32_t rank) {
  const int ptid = threadIdx.x - 32 * NSW, pwarp = ptid >> 5, lane = ptid & 31;
  const int gw = pwarp / (NPW / NGW);
  // A warp converts its eight rows in four steps of 32 pieces (a piece = 16 values of a row = one 16-byte chunk of e4m3).
  // Step `it` of a lane is piece (row, chunk): normally two rows per step, 16 lanes per row.  In CTA 1 of a MODEL1 cache
  // a row has twelve e4m3 chunks and four chunks of 16 bf16 values (two 16-byte loads each), which only change format:
  // there steps 0-2 take the 96 e4m3 pieces in row order and step 3 the 32 bf16 pieces, so that no step mixes the two.
  const bool m1_split = p.m1 && rank == 1;
  auto piece_row = [&](int it) -> uint32_t {
    if (m1_split) return (uint32_t)PROWS * pwarp + (it < 3 ? (uint32_t)(32 * it + lane) / 12u : (uint32_t)lane >> 2);
    return (uint32_t)PROWS * pwarp + 2 * it + (lane >> 4);
  };
  auto piece_ch = [&](int it) -> uint32_t {
    if (m1_split) return it < 3 ? (uint32_t)(32 * it + lane) % 12u : 12u + ((uint32_t)lane & 3u);
    return (uint32_t)lane & 15u;
  };
  auto m1_bf16 = [&](int it) { return m1_split && it == 3; };
  // A piece becomes two 16-byte chunks of a stage row, stored by two instructions.  The eight lanes that a 16-byte store
  // instruction serves per cycle hold the pieces of two panels at the same four chunk positions, so if every lane
  // stored its lower chunk first they would hit four of the eight bank groups twice; the lanes of the odd panels
  // therefore store their upper chunk first (they swap the halves of their input and the two chunk positions).
  const uint32_t flip = m1_split ? 0u : ((uint32_t)lane >> 2) & 1u;
  uint32_t total_blocks = 0;
  {
    Item it;
    for (int i = 0; get_item(p, rec, i, it); ++i) total_blocks += (uint32_t)num_blocks(it);
  }
  bool clipped = false;      // a scale beyond what the fp16 stage can hold was met (the values were clipped)
  uint32_t pos = 0;          // ring position
  int item = 0, n = 0, nb = 0;
  for (uint32_t g = 0; g < total_blocks; ++g, ++pos) {
    if (n == 0) {            // first block of an item: its Q goes into the two ring positions before
      Item it;
      get_item(p, rec, item, it);
      nb = num_blocks(it);
      if (!fill_q_positions(p, c, rank, pwarp, lane, item, it.sq, it.req, pos)) return;
    }
    if (++n >= nb) { n = 0; ++item; }
    const int st = pos % NSTAGE_DECODE, slot = g % NRAW;
    bool ok = wait(c, RAW_FULL + gw * NRAW + slot, g / NRAW, 14);
    if (!__all_sync(0xffffffffu, ok)) return;
    const uint32_t raw = c.base + SM_RAW + (uint32_t)slot * RAW_BYTES, stage = stage_addr(c, st);
    // all loads first, then the arithmetic, then the stores: the shared-memory accesses are ordered among themselves,
    // so this order is what lets the four chunks overlap
    uint4 in[PROWS / 2], in2[PROWS / 2];
    uint32_t sc_bits[PROWS / 2];
#pragma unroll
    for (int it = 0; it < PROWS / 2; ++it) {
      const uint32_t row = piece_row(it), ch = piece_ch(it);
      if (p.m1) {
        if (m1_bf16(it)) {
          in[it] = lds_16(raw + M1_RAW_ROPE + row * 128u + (ch - 12) * 32u);
          in2[it] = lds_16(raw + M1_RAW_ROPE + row * 128u + (ch - 12) * 32u + 16u);
          sc_bits[it] = 127u;
        } else {
          in[it] = lds_16(raw + row * (rank == 0 ? 256u : 192u) + ch * 16u);
          asm volatile("ld.shared.u8 %0, [%1];" : "=r"(sc_bits[it]) : "r"(raw + M1_RAW_SCALE + row * 8u + 4u * rank + (ch >> 2)));
        }
      } else {
        const uint32_t sc = raw + RAW_SCALE + (row >> 2) * SCALE_GROUP + (row & 3u) * 16u;
        in[it] = lds_16(raw + RAW_NOPE + row * 256u + ch * 16u);
        if (p.layout == FMLA_LAYOUT_V32) sc_bits[it] = lds_u32(sc + 4u * (2u * rank + (ch >> 3)));
        else asm volatile("ld.shared.u8 %0, [%1];" : "=r"(sc_bits[it]) : "r"(sc + 8u * rank + (ch >> 1)));
      }
    }
    const uint32_t rrow = (uint32_t)PROWS * pwarp + (lane >> 2), chr = lane & 3;
    uint4 rope = make_uint4(0u, 0u, 0u, 0u);
    if (!p.m1) rope = lds_16(raw + RAW_ROPE + (rrow >> 2) * ROPE_GROUP + (rrow & 3u) * 64u + chr * 16u);
    uint4 lo[PROWS / 2], hi[PROWS / 2];
    auto convert_piece = [&](int it) {
      if (m1_bf16(it)) {      // bf16 -> fp16: values beyond fp16's range saturate and are reported
        uint32_t amax = 0;
        const uint32_t w[8] = {in[it].x, in[it].y, in[it].z, in[it].w, in2[it].x, in2[it].y, in2[it].z, in2[it].w};
        uint32_t o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) { amax = absmax_bf16x2(amax, w[k]); o[k] = bf16x2_to_f16x2(w[k]); }
        clipped |= beyond_f16(amax);
        lo[it] = make_uint4(o[0], o[1], o[2], o[3]);
        hi[it] = make_uint4(o[4], o[5], o[6], o[7]);
        return;
      }
      const float scale = p.layout == FMLA_LAYOUT_V32 ? __uint_as_float(sc_bits[it]) : e8m0_to_float(sc_bits[it]);
      clipped |= scale > MAX_STAGED_SCALE;
      const uint4 src = flip ? make_uint4(in[it].z, in[it].w, in[it].x, in[it].y) : in[it];
      dequant_chunk_f16(src, scale_to_half2(scale), lo[it], hi[it]);
    };
    auto store_piece = [&](int it) {
      const uint32_t row = piece_row(it), ch = piece_ch(it);
      const uint32_t panel = stage + (ch >> 2) * PANEL;
      const uint32_t f = m1_bf16(it) ? 0u : flip;
      st_shared16(panel + swz(row, 2 * (ch & 3) + f), lo[it]);
      st_shared16(panel + swz(row, 2 * (ch & 3) + 1 - f), hi[it]);
    };
    // Two halves: the stores of the first two pieces are under way while the last two are converted.  Only the stores
    // need the stage: what comes before them overlaps the products that still read its previous contents.
    convert_piece(0);
    convert_piece(1);
    const uint32_t use = pos / NSTAGE_DECODE;
    ok = use == 0 || wait(c, KV_EMPTY + st, use - 1, 15);
    if (!__all_sync(0xffffffffu, ok)) return;
    store_piece(0);
    store_piece(1);
    convert_piece(2);
    convert_piece(3);
    store_piece(2);
    store_piece(3);
    if (!p.m1) st_shared16(stage + ROPE_PANEL + rrow * 64u + ((chr ^ ((rrow >> 1) & 3u)) << 4), rope);
    // the dequantised rows (generic proxy) become visible to the MMAs, and this warp's reads of the raw slot
    // are ordered before the TMA writes of the slot's next use
    fence_async_smem();
    __syncwarp();
    if (lane == 0) {
      mbar_arrive(bar_addr(c, RAW_EMPTY + gw * NRAW + slot));
      arrive_leader(c, KV_FULL + st);
    }
  }
  if (__any_sync(0xffffffffu, clipped) && lane == 0 && c.status) atomicCAS(c.status, 0, FMLA_STATUS_CLIPPED);
}

// ---- MMA issuers (one warp each, CTA 0) ---------------------------------------------------------
// An issuer is a whole warp that stays converged: every lane waits on the barriers and computes the same descriptors,
// and one elected lane issues (see umma_ts_pair_elect for why).
// QK^T issuer k writes S buffer k: it takes the blocks whose running number has parity k, so consecutive blocks are
// issued by two warps and the instruction issue of one overlaps the other's; a block's 20 products still come from
// one thread in a fixed order, which keeps the results bitwise repeatable.
template <class P>
__device__ void issue_qk(const P& p, const SchedRecord& rec, const Ctx& c, uint32_t tmem, uint32_t k) {
  constexpr uint32_t ALL = 0xffffffffu;
  // decode: NoPE k-steps are fp16 x fp16 (Q converted on load, K dequantised to fp16); RoPE k-steps are bf16
  const uint32_t idesc_nope = p.raw ? idesc_16bit(128, 2 * T, 0, 0, false, false) : idesc_bf16(128, 2 * T, false, false);
  constexpr uint32_t idesc_rope = idesc_bf16(128, 2 * T, false, false);
  // RoPE k-steps take Q from shared memory, where both lane halves of the accumulator would see the same 16 features;
  // the products of feature half 0 therefore leave lanes 64-127 untouched and those of half 1 lanes 0-63
  const uint32_t F = 0xffffffffu;
  const uint32_t keep_upper[8] = {0u, 0u, F, F, 0u, 0u, F, F}, keep_lower[8] = {F, F, 0u, 0u, F, F, 0u, 0u};
  const int nst = num_stages(p);
  const uint32_t s_tmem = tmem + TM_S + 64u * k;
  const uint64_t qr0 = smem_desc_kmajor(c.base + SM_QROPE);
  Item it;
  uint32_t seq = 0;
  for (int i = 0; get_item(p, rec, i, it); ++i) {
    if (!__all_sync(ALL, wait(c, Q_FULL, i, 21))) return;
    const uint32_t seq_end = seq + (uint32_t)num_blocks(it);
    for (seq += (seq ^ k) & 1u; seq < seq_end; seq += 2) {
      const uint32_t pos = seq + 2u * (uint32_t)(i + 1);       // ring position: two per item hold its Q
      const int s = pos % nst;
      if (!__all_sync(ALL, wait(c, KV_FULL + s, pos / nst, 22))) return;
      if (seq >= 2 && !__all_sync(ALL, wait(c, S_EMPTY + k, (seq >> 1) - 1, 23))) return;
      tc_fence_after_sync();
      const uint64_t b0 = smem_desc_kmajor(stage_addr(c, s));
      const uint64_t r0 = smem_desc_kmajor_sw64(stage_addr(c, s) + ROPE_PANEL);
#pragma unroll
      for (int j = 0; j < 16; ++j)
        umma_ts_pair_elect(s_tmem, tmem + TM_Q + 8 * j, b0 + (((j >> 2) * PANEL + (j & 3) * 32) >> 4), idesc_nope, j > 0);
      if (!p.m1 && p.d_qk == D_QK) {   // rows of 512 values (MODEL1 decode: the RoPE part is among them as fp16; prefill with d_qk = 512: it reads as zero)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          umma_ss_pair_masked_elect(s_tmem, qr0 + ((j * 32) >> 4), r0 + ((j * 32) >> 4), idesc_rope, true, keep_upper);
          umma_ss_pair_masked_elect(s_tmem, qr0 + (((2 + j) * 32) >> 4), r0 + ((j * 32) >> 4), idesc_rope, true, keep_lower);
        }
      }
      umma_commit_pair_elect(bar_addr(c, S_FULL + k), 0x3);
    }
    seq = seq_end;
  }
}

template <class P>
__device__ void issue_pv(const P& p, const SchedRecord& rec, const Ctx& c, uint32_t tmem) {
  constexpr uint32_t ALL = 0xffffffffu;
  const uint32_t idesc = p.raw ? idesc_16bit(128, 256, 0, 0, false, true) : idesc_bf16(128, 256, false, true);
  const int nst = num_stages(p);
  Item it;
  uint32_t seq = 0;
  for (int i = 0; get_item(p, rec, i, it); ++i) {
    const int nb = num_blocks(it);
    // the item's first product overwrites O: the epilogue of the item before has read it
    if (i > 0 && !__all_sync(ALL, wait(c, O_FREE, i - 1, 33))) return;
    for (int n = 0; n < nb; ++n, ++seq) {
      const uint32_t pos = seq + 2u * (uint32_t)(i + 1);
      const int s = pos % nst, b = seq & 1;
      if (!__all_sync(ALL, wait(c, P_FULL + b, seq >> 1, 31))) return;
      if (!__all_sync(ALL, wait(c, KV_FULL + s, pos / nst, 32))) return;
      tc_fence_after_sync();
      const uint64_t a0 = smem_desc_kmajor(c.base + SM_P + b * P_BYTES);
      const uint64_t v0 = smem_desc_mnmajor(stage_addr(c, s), PANEL);
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int ks = 0; ks < T / 16; ++ks)
          umma_ss_pair_elect(tmem + TM_O + 128 * h, a0 + ((ks * 32) >> 4), v0 + ((h * 2 * PANEL + ks * 2048) >> 4), idesc,
                             n > 0 || ks > 0);
      umma_commit_pair_elect(bar_addr(c, KV_EMPTY + s), 0x3);
      umma_commit_pair_elect(bar_addr(c, PV_DONE + b), 0x3);
    }
  }
}


// ---- softmax / epilogue warps ------------------------------------------------------------------------
// Thread l of the 256 softmax threads works on tensor-memory lane L = l % 128 (head L % 64, feature half
// L / 64 of the dual GEMM) and on column group g = l / 128 (tokens 32g .. 32g+31 of the block, columns
// 128g .. 128g+127 of O).  The four threads of a head (two halves x two column groups) sit in four warps:
//   * a "pair" (same g, the two halves) adds its partial dot products through shared memory: barrier 3 + 2g + (warp & 1);
//   * the "quad" exchanges row maxima and row sums: barrier 1 + (warp & 1).
// All four execute the same sequence of mbarrier waits on the same phases and take the same data-dependent
// decisions (they see the same row maxima), so they reach every named barrier together; a warp that leaves
// because the kernel is aborting keeps arriving on its barriers (leave_group) so that the others cannot block.
__device__ __forceinline__ void pair_sync(int warp) { asm volatile("bar.sync %0, 64;" ::"r"(3 + 2 * (warp >> 2) + (warp & 1)) : "memory"); }
__device__ __forceinline__ void quad_sync(int warp) { asm volatile("bar.sync %0, 128;" ::"r"(1 + (warp & 1)) : "memory"); }
__device__ __noinline__ void leave_group(uint32_t leave_word, int warp) {
  // Named barriers have no time-out, so a leaving warp keeps feeding the three barriers it takes part in (its pair,
  // its quad and the all-warps barrier of the Q hand-over) until every softmax warp of the CTA has left or a bound is
  // reached: whoever still waits in one of them is released, meets the abort flag at its next mbarrier wait and ends
  // up here too.
  __syncwarp();
  if ((threadIdx.x & 31) == 0) asm volatile("red.shared.add.u32 [%0], 1;" ::"r"(leave_word) : "memory");
  for (int it = 0; it < (1 << 16); ++it) {
    asm volatile("bar.arrive %0, 64;" ::"r"(3 + 2 * (warp >> 2) + (warp & 1)) : "memory");
    asm volatile("bar.arrive %0, 128;" ::"r"(1 + (warp & 1)) : "memory");
    asm volatile("bar.arrive 9, 256;" ::: "memory");
    uint32_t left;
    asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(left) : "r"(leave_word));
    if (left >= (uint32_t)NSW) break;
    __nanosleep(200);
  }
}

// packed fp32 arithmetic (two lanes per instruction): the softmax chain is bound by the instructions it issues
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  float2 r;
  asm("{\n\t.reg .b64 ra, rb, rc;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tadd.rn.f32x2 rc, ra, rb;\n\tmov.b64 {%0, %1}, rc;\n\t}"
      : "=f"(r.x), "=f"(r.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return r;
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 r;
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\tfma.rn.f32x2 rd, ra, rb, rc;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(r.x), "=f"(r.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return r;
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// Q of one query -> tensor memory (NoPE) and shared memory (RoPE) with plain loads.  Lanes 0-63 take Q[head, NoPE 0:256],
// lanes 64-127 take Q[head, NoPE 256:512]; column c of the Q region holds elements (2c, 2c+1) of the lane's 256.
// Column group g of a lane loads NoPE columns 64g .. 64g+63; the thread also writes RoPE dims 32 half + 16 g .. + 15
// of its head into the 128B-swizzled RoPE panel.
template <class P>
__device__ __forceinline__ void load_q_to_tmem(const P& p, const Ctx& c, const Item& it, uint32_t tmem_lane, int head, int h, int half, int g, uint32_t& qmax) {
  const __nv_bfloat16* row = it.q + (int64_t)head * p.q_stride_h;
  const __nv_bfloat16* nope = row + 256 * half + 128 * g;
  const __nv_bfloat16* rope = row + 512 + 32 * half + 16 * g;
  uint4 a[8], b[8], e[2];
  if (head < p.h_q) {
#pragma unroll
    for (int k = 0; k < 8; ++k) a[k] = ldg_nc_16(nope + 8 * k);
#pragma unroll
    for (int k = 0; k < 8; ++k) b[k] = ldg_nc_16(nope + 64 + 8 * k);
    e[0] = e[1] = make_uint4(0u, 0u, 0u, 0u);
    if (p.d_qk == D_QK) {     // rows of 512 values end here: their RoPE part reads as zero
      e[0] = ldg_nc_16(rope);
      e[1] = ldg_nc_16(rope + 8);
    }
  } else {      // a head of the padding of a 64-head group: zeros
#pragma unroll
    for (int k = 0; k < 8; ++k) a[k] = b[k] = make_uint4(0u, 0u, 0u, 0u);
    e[0] = e[1] = make_uint4(0u, 0u, 0u, 0u);
  }
  uint32_t r[32];
#pragma unroll
  for (int k = 0; k < 8; ++k) { r[4 * k] = a[k].x; r[4 * k + 1] = a[k].y; r[4 * k + 2] = a[k].z; r[4 * k + 3] = a[k].w; }
  if (p.raw) {   // decode over FP8 caches multiplies the NoPE part in fp16
#pragma unroll
    for (int k = 0; k < 32; ++k) { qmax = absmax_bf16x2(qmax, r[k]); r[k] = bf16x2_to_f16x2(r[k]); }
  }
  tmem_st32(tmem_lane + TM_Q + 64 * g, r);
#pragma unroll
  for (int k = 0; k < 8; ++k) { r[4 * k] = b[k].x; r[4 * k + 1] = b[k].y; r[4 * k + 2] = b[k].z; r[4 * k + 3] = b[k].w; }
  if (p.raw) {
#pragma unroll
    for (int k = 0; k < 32; ++k) { qmax = absmax_bf16x2(qmax, r[k]); r[k] = bf16x2_to_f16x2(r[k]); }
  }
  tmem_st32(tmem_lane + TM_Q + 64 * g + 32, r);
  st_shared16(c.base + SM_QROPE + swz(h, 4 * half + 2 * g), e[0]);
  st_shared16(c.base + SM_QROPE + swz(h, 4 * half + 2 * g + 1), e[1]);
  fence_async_smem();      // the panel is read by the MMAs (async proxy)
  tmem_st_wait();
}
// Q of one query from its two ring positions (see fill_q_positions) into tensor memory (NoPE) and into the RoPE panel.
// `src` is the stage that holds this thread's feature half.  The thread copies, of each of the four NoPE tiles, the 32
// dims of its column group to its tensor-memory lane, and the 16 RoPE dims 32 half + 16 g of its head.
template <class P>
__device__ __forceinline__ void copy_q_from_stage(const P& p, const Ctx& c, uint32_t src, uint32_t tmem_lane, int h, int half, int g, uint32_t& qmax) {
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    uint32_t v[16];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint4 t = lds_16(src + r * PANEL + swz(h, 4 * g + k));
      v[4 * k] = t.x; v[4 * k + 1] = t.y; v[4 * k + 2] = t.z; v[4 * k + 3] = t.w;
    }
    if (p.raw) {   // decode over FP8 caches multiplies the NoPE part in fp16
#pragma unroll
      for (int k = 0; k < 16; ++k) { qmax = absmax_bf16x2(qmax, v[k]); v[k] = bf16x2_to_f16x2(v[k]); }
    }
    tmem_st16(tmem_lane + TM_Q + 32 * r + 16 * g, v);
  }
  const uint32_t rp = src + ROPE_PANEL + (uint32_t)h * 64u, sw = ((uint32_t)h >> 1) & 3u;
  const uint4 e0 = lds_16(rp + (((uint32_t)(2 * g) ^ sw) << 4)), e1 = lds_16(rp + (((uint32_t)(2 * g + 1) ^ sw) << 4));
  st_shared16(c.base + SM_QROPE + swz(h, 4 * half + 2 * g), e0);
  st_shared16(c.base + SM_QROPE + swz(h, 4 * half + 2 * g + 1), e1);
  // the panel is read by the MMAs (async proxy), and this thread's reads of the stages come before the TMA writes of
  // their next use
  fence_async_smem();
  tmem_st_wait();
}

// Asks L2 for the part of a query's Q row that load_q_to_tmem will read.
template <class P>
__device__ __forceinline__ void prefetch_q(const P& p, const Item& it, int head, int half, int g) {
  if (head >= p.h_q) return;
  const __nv_bfloat16* row = it.q + (int64_t)head * p.q_stride_h;
  const __nv_bfloat16* nope = row + 256 * half + 128 * g;
  asm volatile("prefetch.global.L2 [%0];" ::"l"(nope));
  asm volatile("prefetch.global.L2 [%0];" ::"l"(nope + 64));
  if (p.d_qk == D_QK) asm volatile("prefetch.global.L2 [%0];" ::"l"(row + 512 + 32 * half + 16 * g));
}

template <class P>
__device__ void softmax_role(const P& p, const SchedRecord& rec, const Ctx& c, uint32_t tmem, uint32_t rank) {
  const int l = threadIdx.x;                 // 0..255
  const int warp = l >> 5, lane = l & 31;
  const int L = l & 127, team = l >> 7;      // tensor-memory lane, softmax team
  const int h = L & 63, half = L >> 6;
  const int g = team;                        // column group of this thread in the Q load and the epilogue
  const int slot = 2 * team + half;          // this thread's place among the four threads of head h
  const int head = blockIdx.z * 128 + (int)rank * 64 + h;
  const uint32_t tmem_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
  // Exchange buffer: region r (the receiving feature half) holds 64 rows (heads) of 32 floats; the 16-byte chunk k
  // of row h sits at chunk position k ^ (h & 7), which spreads eight consecutive rows over all bank groups.
  // The 32 partial sums a thread hands to its mate travel in two halves of 16: one through the exchange buffer and
  // one through the team's own P buffer, which is idle until the block's probabilities are written.  Both are laid out
  // as [head range h / 32][receiving half][32 heads][16 floats]: the 4 KB of a head range are exactly the P rows of the
  // same 32 heads, so only the two warps of a pair ever touch them, in the exchange as well as when P is written.  The
  // 16-byte chunk k of a 64-byte row sits at chunk position k ^ ((row / 2) % 4): eight consecutive rows then cover all
  // bank groups.  (Decode has no shared memory to spare for this; prefill has, and gives the second half a buffer like
  // the first one, so that a block need not wait at its start for the PV product that read the P buffer last.)
  const uint32_t xoff = 4096u * (uint32_t)(h >> 5) + 64u * (uint32_t)(h & 31);
  const uint32_t xput = 2048u * (uint32_t)(1 - half) + xoff, xget = 2048u * (uint32_t)half + xoff;
  const uint32_t xsw = ((uint32_t)h >> 1) & 3u;
  const uint32_t pbuf = c.base + SM_P + team * P_BYTES, xbuf = c.base + SM_XCHG;
  const uint32_t xbuf2 = p.raw ? pbuf : c.base + SM_XCHG2;
  const uint32_t max_mine = c.base + SM_MAX + 4u * (64 * slot + h), max_mate = c.base + SM_MAX + 4u * (64 * (slot ^ 1) + h);
  const uint32_t mref_mine = c.base + SM_MREF + 4u * (64 * team + h), mref_other = c.base + SM_MREF + 4u * (64 * (team ^ 1) + h);
  const uint32_t sum_base = c.base + SM_SUM + 4u * h, mtrue_base = c.base + SM_MTRUE + 4u * h;
  const bool real_head = head < p.h_q;     // h_q = 64 (mod 128): the last group's upper 64 heads are padding (Q = 0, nothing stored)
  const float sink2 = p.attn_sink && real_head ? __ldg(p.attn_sink + head) * LOG2E : -CUDART_INF_F;
  const uint32_t leave_word = c.base + SM_LEAVE;

  Item it, it_next;
  bool have = get_item(p, rec, 0, it);
  const int nst = num_stages(p);
  uint32_t q_absmax = 0;                     // decode: largest |q| of the NoPE part seen by this thread (Q is staged in fp16)
  // Q of the pair's `index`-th item, which lies in ring positions pos and pos + 1, goes to tensor memory and to the
  // RoPE panel; the caller has made sure that no QK^T product that reads the Q before is still running.  Then the two
  // stages are handed back: the team that comes `early` only reports at the barrier of all softmax warps, the other
  // one waits there and its first thread releases the stages.  Returns false when aborting.
  auto take_q = [&](const Item& q_it, int index, uint32_t pos, bool early) -> bool {
    const bool ok = wait(c, QL_FULL + (index & 1), index >> 1, 48);
    if (!__all_sync(0xffffffffu, ok)) return false;
    if (p.q_tma) copy_q_from_stage(p, c, stage_addr(c, (int)((pos + (uint32_t)half) % (uint32_t)nst)), tmem_lane, h, half, g, q_absmax);
    else load_q_to_tmem(p, c, q_it, tmem_lane, head, h, half, g, q_absmax);
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) arrive_leader(c, Q_FULL);
    if (early) {
      asm volatile("bar.arrive 9, 256;" ::: "memory");
    } else {
      asm volatile("bar.sync 9, 256;" ::: "memory");
      if (L == 0) {
        mbar_arrive(bar_addr(c, KV_EMPTY + (int)(pos % (uint32_t)nst)));
        mbar_arrive(bar_addr(c, KV_EMPTY + (int)((pos + 1u) % (uint32_t)nst)));
      }
    }
    return true;
  };
  if (have && !take_q(it, 0, 0u, team == 0)) { leave_group(leave_word, warp); return; }
  uint32_t seq0 = 0;                         // number of blocks of the items before this one
  for (int i = 0; have; ++i) {
    const bool have_next = get_item(p, rec, i + 1, it_next);
    if (have_next && !p.q_tma) prefetch_q(p, it_next, head, half, g);
    // m_mine: the reference maximum that l_sum is relative to; m_true: largest logit (base 2) of this team's blocks
    float m_mine = -CUDART_INF_F, m_true = -CUDART_INF_F, l_sum = 0.f;
    const uint32_t seq_end = seq0 + (uint32_t)num_blocks(it);
    for (uint32_t seq = seq0 + ((seq0 ^ (uint32_t)team) & 1u); seq < seq_end; seq += 2) {
      bool ok = wait(c, S_FULL + team, seq >> 1, 41);
      // the other team has finished with the exchange buffer and has settled the reference maximum of block seq - 1
      ok = ok && (seq == 0 || wait(c, DEC + (team ^ 1), (seq - 1) >> 1, 42));
      // decode: the PV product that read this team's P buffer last has completed (it did so about a block ago): the
      // buffer carries half of the exchange now and the block's probabilities later
      if (p.raw) ok = ok && (seq < 2 || wait(c, PV_DONE + team, (seq >> 1) - 1, 45));
      if (!__all_sync(0xffffffffu, ok)) { leave_group(leave_word, warp); return; }
      tc_fence_after_sync();
      // of the block's 64 tokens this thread finishes 32 (tokens 32*half ..): it reads its own partial dot
      // products of the other 32 ("send"), which go to its mate in the other feature half, and of its own ("keep")
      uint32_t keep[32];
      {
        uint32_t send[32];
        tmem_ld32(tmem_lane + TM_S + 64 * team + 32 * (1 - half), send);
        tmem_ld32(tmem_lane + TM_S + 64 * team + 32 * half, keep);      // both loads in flight together
        tmem_ld_wait();
#pragma unroll
        for (int k = 0; k < 8; ++k)
          st_shared16((k < 4 ? xbuf : xbuf2) + xput + (((uint32_t)(k & 3) ^ xsw) << 4),
                      make_uint4(send[4 * k], send[4 * k + 1], send[4 * k + 2], send[4 * k + 3]));
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) arrive_leader(c, S_EMPTY + team);
      pair_sync(warp);
      float x[32];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint4 t = lds_16((k < 4 ? xbuf : xbuf2) + xget + (((uint32_t)(k & 3) ^ xsw) << 4));
        const float2 lo = add2(make_float2(__uint_as_float(keep[4 * k]), __uint_as_float(keep[4 * k + 1])), make_float2(__uint_as_float(t.x), __uint_as_float(t.y)));
        const float2 hi = add2(make_float2(__uint_as_float(keep[4 * k + 2]), __uint_as_float(keep[4 * k + 3])), make_float2(__uint_as_float(t.z), __uint_as_float(t.w)));
        x[4 * k] = lo.x; x[4 * k + 1] = lo.y; x[4 * k + 2] = hi.x; x[4 * k + 3] = hi.y;
      }
      const uint32_t vmask = lds_u32(c.base + SM_MASK + 8u * (seq % RING) + 4u * half);
      float mx = -CUDART_INF_F;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        x[j] = (vmask >> j) & 1u ? x[j] : -CUDART_INF_F;
        mx = fmaxf(mx, x[j]);
      }
      mx *= p.scale_log2;                                  // the scale is positive: max commutes with it
      sts_f32(max_mine, mx);
      pair_sync(warp);
      mx = fmaxf(mx, lds_f32(max_mate));                   // maximum of the block's 64 tokens for this head
      m_true = fmaxf(m_true, mx);

      // The reference maximum moves lazily: only when the block maximum exceeds it by more than the threshold.  The
      // two teams take turns, so the value before this block is the one the other team left after block seq - 1
      // (-inf at the first block of a query); the two threads of a head in this team take the same decision.
      const float m_prev = seq == seq0 ? -CUDART_INF_F : lds_f32(mref_other);
      const bool bump = mx > m_prev + RESCALE_THRESHOLD || (m_prev == -CUDART_INF_F && mx != -CUDART_INF_F);
      const float m_new = bump ? mx : m_prev;
      const float alpha = !bump ? 1.f : (m_prev == -CUDART_INF_F ? 0.f : exp2f(m_prev - mx));
      if (half == 0) sts_f32(mref_mine, m_new);
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_addr(c, DEC + team));
      if (__any_sync(0xffffffffu, bump && alpha != 0.f)) {   // rescale this lane's 256 columns of O
        // every PV product issued so far must have completed.  This team's previous one first (decode has waited for it
        // at the top of the block): then the product before that one has completed too, and the parity of the other
        // team's barrier cannot be mistaken for that earlier completion
        ok = p.raw || seq < 2 || wait(c, PV_DONE + team, (seq >> 1) - 1, 45);
        ok = ok && wait(c, PV_DONE + (team ^ 1), (seq - 1) >> 1, 44);
        if (!__all_sync(0xffffffffu, ok)) { leave_group(leave_word, warp); return; }
        tc_fence_after_sync();
#pragma unroll 1
        for (int ch = 0; ch < 8; ++ch) {
          uint32_t o[32];
          tmem_ld32(tmem_lane + TM_O + 32 * ch, o);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
          tmem_st32(tmem_lane + TM_O + 32 * ch, o);
        }
        tmem_st_wait();
      }
      if (m_new != m_mine) { l_sum *= exp2f(m_mine - m_new); m_mine = m_new; }   // m_mine = -inf: l_sum is 0 and stays 0

      // p = 2^(x * scale - m_ref); while no valid token has been seen every x is -inf and the offset is 0, so p = 0
      const float off = m_new == -CUDART_INF_F ? 0.f : -m_new;
      uint32_t pk[16];
      float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), off2 = make_float2(off, off);
      // P rows of these 32 heads overwrite the pair's exchange data in the buffer: the pair barrier above (row maxima)
      // lies between the mate's reads of that data and these stores.  Prefill has not waited yet for the PV product that
      // read the buffer last.  Each 16-byte chunk is stored as soon as its eight probabilities exist, so that the stores
      // travel under the remaining exponentials.
      if (!p.raw) {
        ok = seq < 2 || wait(c, PV_DONE + team, (seq >> 1) - 1, 45);
        if (!__all_sync(0xffffffffu, ok)) { leave_group(leave_word, warp); return; }
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float2 a = fma2(make_float2(x[2 * j], x[2 * j + 1]), scale2, off2);
        const float2 e = make_float2(exp2f(a.x), exp2f(a.y));
        sum2[j & 1] = add2(sum2[j & 1], e);
        pk[j] = p.raw ? pack_f16x2(e.x, e.y) : pack_bf16x2(e.x, e.y);
        if ((j & 3) == 3) st_shared16(pbuf + swz(h, 4 * half + (j >> 2)), make_uint4(pk[j - 3], pk[j - 2], pk[j - 1], pk[j]));
      }
      l_sum += (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y);

      fence_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) arrive_leader(c, P_FULL + team);
    }
    seq0 = seq_end;
    const uint32_t last = seq_end - 1;        // the query's last block

    // ---- end of the item: epilogue (columns 128g .. 128g+127 of the lane's 256) and the next query's Q ----
    float mul = 0.f, lse2 = 0.f, m_fin = 0.f;
    bool empty = true;
    float* dst_f32 = nullptr;
    __nv_bfloat16* dst_bf16 = nullptr;
    const bool mine_last = (last & 1u) == (uint32_t)team;     // this team took the query's last block
    auto epi_begin = [&]() -> bool {            // row sums and maxima of the quad, output scale, destination
      // the query's final reference maximum is the one the last block's team has settled
      bool ok = mine_last || wait(c, DEC + (team ^ 1), last >> 1, 43);
      if (!__all_sync(0xffffffffu, ok)) return false;
      m_fin = lds_f32(c.base + SM_MREF + 4u * (64 * (last & 1u) + h));
      sts_f32(sum_base + 256u * slot, m_mine == m_fin ? l_sum : l_sum * exp2f(m_mine - m_fin));
      if (half == 0) sts_f32(mtrue_base + 256u * team, m_true);   // the two halves of a team hold the same value
      ok = wait(c, PV_DONE + (last & 1), last >> 1, 47);
      if (!__all_sync(0xffffffffu, ok)) return false;
      tc_fence_after_sync();
      quad_sync(warp);
      const float l_tot = (lds_f32(sum_base) + lds_f32(sum_base + 256u)) + (lds_f32(sum_base + 512u) + lds_f32(sum_base + 768u));
      m_true = fmaxf(lds_f32(mtrue_base), lds_f32(mtrue_base + 256u));
      empty = l_tot == 0.f;
      lse2 = empty ? -CUDART_INF_F : m_fin + log2f(l_tot);
      if (it.split) mul = empty ? 0.f : 1.f / l_tot;
      else mul = empty ? 0.f : 1.f / (l_tot + exp2f(sink2 - m_fin));
      const int col0 = 256 * half + 128 * g;
      if (it.split) dst_f32 = p.o_accum + (it.row + head) * D_V + col0;
      else if (p.mode == 0) dst_bf16 = p.out + it.req * p.o_stride0 + it.sq * p.o_stride1 + head * p.o_stride_h + col0;
      else dst_bf16 = p.out + (it.row * p.h_q + head) * D_V + col0;
      return true;
    };
    // A plain store of a warp would touch 32 rows of the output with 16 bytes each, one memory transaction per lane, and
    // the epilogue would cost as much as several blocks.  So the warp stages its 32 heads x 32 columns (x 16 for fp32
    // partial results) in its quarter of the team's P buffer, idle between two queries, in the 64B-swizzled layout of a
    // TMA box, and one lane sends the box off; the buffer is rewritten once the previous box has been read.  The quarter
    // lies in the 4 KB that the warp shares with the other warp of its pair in the block loop (see xoff), and the pair
    // meets after its last boxes have been read, before either goes back to the block loop.
    const uint32_t scratch = pbuf + 4096u * (uint32_t)(warp & 1) + 2048u * (uint32_t)((warp >> 1) & 1), scratch_row = scratch + (uint32_t)lane * 64u;
    const uint32_t scratch_sw = ((uint32_t)lane >> 1) & 3u;
    const int head_warp = head - lane;          // first head of this warp
    // The four chunks of 32 columns through the staging buffer: the next chunk's tensor-memory load is issued before
    // the current chunk waits for the buffer, so that the two latencies overlap.
    auto epi_chunks_tma = [&]() {
      if (!real_head) return;                   // warp-uniform: a warp's 32 heads lie in one 64-head half
      uint32_t o[2][32];
      const uint32_t src = tmem_lane + TM_O + 128 * g;
      const int col0 = 256 * half + 128 * g;
      const int acc_row = it.split ? (int)(it.row / p.h_q) : 0;
      tmem_ld32(src, o[0]);
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t (&cur)[32] = o[ch & 1];
        tmem_ld_wait();
        if (ch < 3) tmem_ld32(src + 32 * (ch + 1), o[(ch + 1) & 1]);
        if (it.split) {
#pragma unroll
          for (int j = 0; j < 32; ++j) cur[j] = __float_as_uint(__uint_as_float(cur[j]) * mul);
#pragma unroll
          for (int sub = 0; sub < 2; ++sub) {
            if (lane == 0) bulk_wait_read();
            __syncwarp();
#pragma unroll
            for (int k = 0; k < 4; ++k)
              st_shared16(scratch_row + (((uint32_t)k ^ scratch_sw) << 4),
                          make_uint4(cur[16 * sub + 4 * k], cur[16 * sub + 4 * k + 1], cur[16 * sub + 4 * k + 2], cur[16 * sub + 4 * k + 3]));
            fence_async_smem();
            __syncwarp();
            if (lane == 0) { tma_store_4d(&p.map_acc, col0 + 32 * ch + 16 * sub, head_warp, acc_row, 0, scratch); bulk_commit(); }
          }
        } else {
          uint4 v[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            v[k].x = pack_bf16x2(__uint_as_float(cur[8 * k]) * mul, __uint_as_float(cur[8 * k + 1]) * mul);
            v[k].y = pack_bf16x2(__uint_as_float(cur[8 * k + 2]) * mul, __uint_as_float(cur[8 * k + 3]) * mul);
            v[k].z = pack_bf16x2(__uint_as_float(cur[8 * k + 4]) * mul, __uint_as_float(cur[8 * k + 5]) * mul);
            v[k].w = pack_bf16x2(__uint_as_float(cur[8 * k + 6]) * mul, __uint_as_float(cur[8 * k + 7]) * mul);
          }
          if (lane == 0) bulk_wait_read();
          __syncwarp();
#pragma unroll
          for (int k = 0; k < 4; ++k) st_shared16(scratch_row + (((uint32_t)k ^ scratch_sw) << 4), v[k]);
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_4d(&p.map_out, col0 + 32 * ch, head_warp, p.mode == 0 ? it.sq : (int)it.row, p.mode == 0 ? it.req : 0, scratch);
            bulk_commit();
          }
        }
      }
    };
    auto epi_chunk = [&](int ch) {              // 32 columns of O with plain stores: scale, convert, store
      if (!real_head) return;
      uint32_t o[32];
      tmem_ld32(tmem_lane + TM_O + 128 * g + 32 * ch, o);
      tmem_ld_wait();
      if (it.split) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<float4*>(dst_f32 + 32 * ch + 4 * j) =
              make_float4(__uint_as_float(o[4 * j]) * mul, __uint_as_float(o[4 * j + 1]) * mul,
                          __uint_as_float(o[4 * j + 2]) * mul, __uint_as_float(o[4 * j + 3]) * mul);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 v;
          v.x = pack_bf16x2(__uint_as_float(o[8 * j]) * mul, __uint_as_float(o[8 * j + 1]) * mul);
          v.y = pack_bf16x2(__uint_as_float(o[8 * j + 2]) * mul, __uint_as_float(o[8 * j + 3]) * mul);
          v.z = pack_bf16x2(__uint_as_float(o[8 * j + 4]) * mul, __uint_as_float(o[8 * j + 5]) * mul);
          v.w = pack_bf16x2(__uint_as_float(o[8 * j + 6]) * mul, __uint_as_float(o[8 * j + 7]) * mul);
          *reinterpret_cast<uint4*>(dst_bf16 + 32 * ch + 8 * j) = v;
        }
      }
    };
    auto epi_end = [&]() {
      if (slot != 0 || !real_head) return;
      if (it.split) { p.lse_accum[it.row + head] = lse2; return; }
      const float lse_nat = empty ? CUDART_INF_F : lse2 * LN2;
      if (p.mode == 0) p.lse[it.req * p.lse_stride0 + it.sq * p.lse_stride1 + head] = lse_nat;
      else {
        p.lse[it.row * p.h_q + head] = lse_nat;
        p.max_logits[it.row * p.h_q + head] = empty ? -CUDART_INF_F : m_true * LN2;
      }
    };
    // The next query's Q first: it waits in its ring positions, and once it is in tensor memory the next query's first
    // QK^T products run beside this query's last PV product and the epilogue.  Q may be replaced when every QK^T
    // product of this query is complete: the team that took the last block knows (it has read that S, and the block
    // before was settled before it started); the other team, idle since the block before, waits for the last S without
    // consuming it and moves its share of Q while the last block's softmax runs.
    if (have_next) {
      const bool ok = mine_last || wait(c, S_FULL + (team ^ 1), last >> 1, 46);
      if (!__all_sync(0xffffffffu, ok)) { leave_group(leave_word, warp); return; }
      tc_fence_after_sync();
      if (!take_q(it_next, i + 1, seq_end + 2u * (uint32_t)(i + 1), !mine_last)) { leave_group(leave_word, warp); return; }
    }
    if (!epi_begin()) { leave_group(leave_word, warp); return; }
    if (p.out_tma) epi_chunks_tma();
    else {
#pragma unroll 1
      for (int ch = 0; ch < 4; ++ch) epi_chunk(ch);
    }
    epi_end();
    // O has been read: the next query's first PV product may overwrite it
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) {
      arrive_leader(c, O_FREE);
      if (p.out_tma) bulk_wait_read();          // the P buffer goes back to the block loop
    }
    __syncwarp();
    if (p.out_tma) pair_sync(warp);
    it = it_next;
    have = have_next;
  }
  if (p.out_tma && lane == 0) bulk_wait_all();   // this thread's output boxes are written before the CTA goes
  if (p.raw && __any_sync(0xffffffffu, beyond_f16(q_absmax)) && lane == 0 && c.status) atomicCAS(c.status, 0, FMLA_STATUS_CLIPPED);
}

// ---- kernel ------------------------------------------------------------------------------------------
template <int MODE, int EXTRA>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(threads_of(raw_ring(MODE, EXTRA)), 1)
pair_attn_kernel(const __grid_constant__ ParamsT<MODE, EXTRA> p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  Ctx c;
  c.base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  c.abort_flag = reinterpret_cast<volatile int*>(__cvta_shared_to_generic(c.base + SM_ABORT));
  const uint32_t rank = cluster_ctarank();
  c.peer = rank ^ 1u;
  c.status = p.status;
  const int warp = threadIdx.x >> 5;

  SchedRecord rec;
  rec.begin_req = 0; rec.end_req = -1; rec.begin_block = rec.end_block = rec.begin_split = rec.first_split = rec.last_split = rec.pad = 0;
  if (p.mode == 0) {
    rec = p.sched[blockIdx.x >> 1];
    // decode: the combine kernel that follows in the stream may start launching; it waits for this grid's completion itself
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  }

  if (threadIdx.x == 0) {
    *c.abort_flag = 0;
    sts_u32(c.base + SM_LEAVE, 0u);
    for (int s = 0; s < MAX_STAGES; ++s) {
      mbar_init(bar_addr(c, KV_FULL + s), 2 * NPW);    // the producer warps of both CTAs
      mbar_init(bar_addr(c, KV_EMPTY + s), 1);
    }
    for (int s = 0; s < NGW * NRAW; ++s) {
      mbar_init(bar_addr(c, RAW_FULL + s), 1);               // the gather warp's expect_tx arrival + the bytes
      mbar_init(bar_addr(c, RAW_EMPTY + s), NPW / NGW);      // the converter warps that read this quarter of the slot
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_addr(c, S_FULL + b), 1);
      mbar_init(bar_addr(c, S_EMPTY + b), NSW);              // the warps of one softmax team in both CTAs
      mbar_init(bar_addr(c, P_FULL + b), NSW);
      mbar_init(bar_addr(c, PV_DONE + b), 1);
      mbar_init(bar_addr(c, DEC + b), NSW / 2);              // the warps of one team of this CTA
    }
    mbar_init(bar_addr(c, Q_FULL), 2 * NSW);
    mbar_init(bar_addr(c, O_FREE), 2 * NSW);
    for (int b = 0; b < 2; ++b) mbar_init(bar_addr(c, QL_FULL + b), 2 * 5);   // five fetching warps per ring position (fill_q_positions)
    mbar_init_fence();
  }
  if (warp == QK_WARP) { tmem_alloc<2>(c.base + SM_TMEM, TM_COLS); tmem_relinquish<2>(); }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync();
  tc_fence_after_sync();
  uint32_t tmem;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem) : "r"(c.base + SM_TMEM));

  // The register file is re-divided between the warpgroups (four consecutive warps each): the softmax teams hold a
  // block's 64 partial sums and 32 probabilities per thread, the other roles need few registers.
  if (warp < NSW) {
    reg_inc<REGS_SOFTMAX>();
    softmax_role(p, rec, c, tmem, rank);
  } else if (warp < NSW + NPW) {
    reg_dec<regs_producer(raw_ring(MODE, EXTRA))>();
    if (p.raw) convert_role(p, rec, c, rank);
    else producer_role(p, rec, c, rank);
  } else if (warp < GATHER_WARP) {
    reg_dec<regs_issuer(raw_ring(MODE, EXTRA))>();
    if (rank == 0) {
      if (warp < PV_WARP) issue_qk(p, rec, c, tmem, (uint32_t)(warp - QK_WARP));
      else if (warp == PV_WARP) issue_pv(p, rec, c, tmem);
    }
  } else {
    reg_dec<REGS_GATHER>();
    if (p.raw) gather_role(p, rec, c, rank, warp - GATHER_WARP);
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync();
  if (warp == QK_WARP) tmem_dealloc<2>(tmem, TM_COLS);
}

// q viewed as (576, h_q, n1, n2) with element strides; box = box_cols dims x 64 heads.  Returns false if the driver
// refuses the strides (the kernel then reads Q with plain loads).
static bool make_q_map(CUtensorMap* map, const void* q, int h_q, uint64_t n1, uint64_t n2, int64_t stride_h, int64_t stride1,
                       int64_t stride2, uint32_t box_cols, CUtensorMapSwizzle swizzle, int d_qk = D_QK) {
  if (stride_h <= 0 || stride1 <= 0 || stride2 <= 0) return false;
  const uint64_t dims[4] = {(uint64_t)d_qk, (uint64_t)h_q, n1, n2};
  const uint64_t strides[3] = {(uint64_t)stride_h * 2, (uint64_t)stride1 * 2, (uint64_t)stride2 * 2};
  const uint32_t box[4] = {box_cols, 64, 1, 1};
  return tmap::encode(map, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, dims, strides, box, swizzle) == 0;
}
// An output tensor viewed as (512, h_q, n1, n2) with element strides; box = box_cols dims x 32 heads, 64 bytes wide,
// 64B swizzle.  Returns false if the driver refuses the strides (the epilogue then stores with plain stores).
static bool make_out_map(CUtensorMap* map, const void* base, CUtensorMapDataType dt, int elem_bytes, int h_q, uint64_t n1, uint64_t n2,
                         int64_t stride_h, int64_t stride1, int64_t stride2, uint32_t box_cols) {
  if (stride_h <= 0 || stride1 <= 0 || stride2 <= 0 || n1 == 0 || n2 == 0) return false;
  const uint64_t dims[4] = {(uint64_t)D_V, (uint64_t)h_q, n1, n2};
  const uint64_t strides[3] = {(uint64_t)stride_h * elem_bytes, (uint64_t)stride1 * elem_bytes, (uint64_t)stride2 * elem_bytes};
  const uint32_t box[4] = {box_cols, 32, 1, 1};
  return tmap::encode(map, base, dt, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B) == 0;
}
// 2-D map over `rows` rows of `cols` elements with a row pitch of `pitch_bytes`; one box is `box_cols` elements of one row.
static int make_row_map(CUtensorMap* map, const void* base, CUtensorMapDataType dt, uint64_t cols, uint64_t rows,
                        uint64_t pitch_bytes, uint32_t box_cols, CUtensorMapSwizzle swizzle) {
  const uint64_t dims[2] = {cols, rows};
  const uint64_t strides[1] = {pitch_bytes};
  const uint32_t box[2] = {box_cols, 1};
  const int rc = tmap::encode(map, base, dt, 2, dims, strides, box, swizzle);
  FMLA_REQUIRE(rc >= 0, FMLA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  FMLA_REQUIRE(rc == 0, FMLA_ERR_CUDA, "cuTensorMapEncodeTiled failed with driver error %d", rc);
  return FMLA_OK;
}

// Diagnostic switch (fmla_set_option): read Q with plain loads even when a tensor map could be made, the path that
// otherwise only runs when the driver refuses q's strides.
std::atomic<int> g_plain_q_loads{0};
std::atomic<int> g_plain_stores{0};     // the same for the epilogue: plain stores instead of TMA box stores

template <int MODE, int EXTRA>
static int launch_mode(const Params& p, dim3 grid, cudaStream_t stream) {
  static tmap::PerDeviceOnce once;
  FMLA_CUDA(once.run([] {
    return cudaFuncSetAttribute(pair_attn_kernel<MODE, EXTRA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
  }));
  ParamsT<MODE, EXTRA> pt;
  static_cast<Params&>(pt) = p;
  if (g_plain_q_loads.load(std::memory_order_relaxed)) pt.q_tma = 0;
  if (g_plain_stores.load(std::memory_order_relaxed)) pt.out_tma = 0;
  pair_attn_kernel<MODE, EXTRA><<<grid, threads_of(raw_ring(MODE, EXTRA)), SMEM_BYTES, stream>>>(pt);
  FMLA_CUDA(cudaGetLastError());
  return FMLA_OK;
}
static int launch(const Params& p, dim3 grid, cudaStream_t stream) {
  if (p.mode != 0) return launch_mode<1, 0>(p, grid, stream);
  if (p.block_table != nullptr) return launch_mode<0, 3>(p, grid, stream);
  if (p.layout == FMLA_LAYOUT_MODEL1) return p.has_extra ? launch_mode<0, 4>(p, grid, stream) : launch_mode<0, 2>(p, grid, stream);
  return p.has_extra ? launch_mode<0, 1>(p, grid, stream) : launch_mode<0, 0>(p, grid, stream);
}

}  // namespace tc


void tc_set_plain_q_loads(int on) { tc::g_plain_q_loads.store(on ? 1 : 0, std::memory_order_relaxed); }
void tc_set_plain_stores(int on) { tc::g_plain_stores.store(on ? 1 : 0, std::memory_order_relaxed); }
void tc_map_cache_stats(unsigned long long* hits, unsigned long long* misses) {
  tmap::Cache& c = tmap::cache();
  std::lock_guard<std::mutex> lock(c.mu);
  *hits = c.hits; *misses = c.misses;
}

bool tc_supported(int h_q) { return h_q > 0 && h_q % 64 == 0; }   // 64 (mod 128): the last pair runs half empty

static int sm_count() {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

int tc_decode_plan(int num_sms, int h_q, int s_q, int* num_sm_parts, int* fixed_overhead_blocks, int* block_topk) {
  // One CTA pair per partition; grid = (2 * partitions, s_q, ceil(h_q / 128)) fills the SMs once.
  const int pairs = num_sms / 2;
  int parts = pairs / (s_q * ((h_q + 127) / 128));
  *num_sm_parts = parts < 1 ? 1 : parts;
  *fixed_overhead_blocks = 3;      // Q load + epilogue of one piece cost about three token blocks
  *block_topk = tc::T;
  return FMLA_OK;
}

// Preconditions of the tensor-core decode kernel beyond the head count.
bool tc_decode_supported(const FmlaDecodeArgs& a) {
  auto pool_ok = [](int64_t stride, int64_t blocks, int64_t page) {
    return stride % ROW_BYTES == 0 && (uint64_t)(blocks - 1) * (uint64_t)(stride / ROW_BYTES) + (uint64_t)page <= 0x7fffffffull;
  };
  if (a.layout == FMLA_LAYOUT_MODEL1) {    // data rows at a pitch of 576 bytes
    auto m1_ok = [](int64_t stride, int64_t blocks, int64_t page) {
      return stride % M1_DATA_BYTES == 0 && (uint64_t)(blocks - 1) * (uint64_t)(stride / M1_DATA_BYTES) + (uint64_t)page <= 0x7fffffffull;
    };
    return a.sm_scale > 0.f && m1_ok(a.kv_stride_block, a.num_blocks, a.page_block_size) &&
           (a.extra_kv == nullptr || m1_ok(a.extra_kv_stride_block, a.extra_num_blocks, a.extra_page_block_size));
  }
  if (!(a.sm_scale > 0.f) || !pool_ok(a.kv_stride_block, a.num_blocks, a.page_block_size)) return false;
  return a.extra_kv == nullptr || pool_ok(a.extra_kv_stride_block, a.extra_num_blocks, a.extra_page_block_size);
}

int launch_tc_decode(const FmlaDecodeArgs& a, cudaStream_t stream) {
  tc::Params p = {};
  p.mode = 0;
  const bool m1 = a.layout == FMLA_LAYOUT_MODEL1;
  // MODEL1: q and the cache rows hold 512 values, all of them V.  The kernel treats them as 512 NoPE values (the q map
  // ends at column 512, so the RoPE tiles read as zero and the RoPE products are skipped).
  p.d_qk = m1 ? M1_D_QK : D_QK;
  p.h_q = a.h_q; p.topk = a.topk;
  FMLA_REQUIRE(a.sm_scale > 0.f, FMLA_ERR_UNSUPPORTED, "the tensor-core kernel needs a positive softmax scale (got %g); use FMLA_KERNEL_SIMT", (double)a.sm_scale);
  p.scale_log2 = a.sm_scale * LOG2E;
  p.q = reinterpret_cast<const __nv_bfloat16*>(a.q);
  p.q_stride0 = a.q_stride_b; p.q_stride1 = a.q_stride_s; p.q_stride_h = a.q_stride_h;
  p.q_tma = tc::make_q_map(&p.map_q, a.q, a.h_q, (uint64_t)a.s_q, (uint64_t)a.b, a.q_stride_h, a.q_stride_s, a.q_stride_b, 64, CU_TENSOR_MAP_SWIZZLE_128B, p.d_qk) &&
            tc::make_q_map(&p.map_q_rope, a.q, a.h_q, (uint64_t)a.s_q, (uint64_t)a.b, a.q_stride_h, a.q_stride_s, a.q_stride_b, 32, CU_TENSOR_MAP_SWIZZLE_64B, p.d_qk);
  p.indices = a.indices; p.idx_stride0 = a.idx_stride_b; p.idx_stride1 = a.idx_stride_s;
  p.topk_length = a.topk_length; p.attn_sink = a.attn_sink;
  p.kv_rows = reinterpret_cast<const uint8_t*>(a.kv);
  p.kv_stride_block = a.kv_stride_block; p.page = (int)a.page_block_size; p.layout = a.layout;
  p.total_rows = a.num_blocks * a.page_block_size;
  p.sched = reinterpret_cast<const SchedRecord*>(a.sched_meta); p.num_splits = a.num_splits;
  p.b = a.b; p.s_q = a.s_q;
  p.out = reinterpret_cast<__nv_bfloat16*>(a.out);
  p.o_stride0 = a.o_stride_b; p.o_stride1 = a.o_stride_s; p.o_stride_h = a.o_stride_h;
  p.lse = a.lse; p.lse_stride0 = a.lse_stride_b; p.lse_stride1 = a.lse_stride_s;
  p.o_accum = a.o_accum; p.lse_accum = a.lse_accum;
  p.status = a.status;
  {   // o_accum holds (b + num_sm_parts) * s_q rows of h_q x 512
    const uint64_t acc_rows = (uint64_t)(a.b + a.num_sm_parts) * (uint64_t)a.s_q;
    p.out_tma = tc::make_out_map(&p.map_out, a.out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.h_q, (uint64_t)a.s_q, (uint64_t)a.b, a.o_stride_h, a.o_stride_s, a.o_stride_b, 32) &&
                tc::make_out_map(&p.map_acc, a.o_accum, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a.h_q, acc_rows, 1, D_V, (int64_t)a.h_q * D_V, (int64_t)(acc_rows * a.h_q) * D_V, 16);
  }
  // Rows are addressed as base + row * 656 with a 32-bit row number, so a block stride must be a whole number of rows
  // (the reference has the same requirement, csrc/sm100/decode/head64/kernel.cuh:911-912); tc_decode_supported() tells
  // the caller, which then takes the CUDA-core kernel.
  FMLA_REQUIRE(tc_decode_supported(a), FMLA_ERR_UNSUPPORTED,
               "sparse_decode: the tensor-core kernel needs KV block strides that are multiples of 656 bytes (MODEL1: 576) "
               "and at most 2^31 rows per cache (got strides %lld / %lld)", (long long)a.kv_stride_block, (long long)a.extra_kv_stride_block);
  if (m1) {
    p.rows_per_block = (int)(a.kv_stride_block / M1_DATA_BYTES);
    const uint64_t vrows = (uint64_t)(a.num_blocks - 1) * p.rows_per_block + a.page_block_size;
    if (int rc = tc::make_row_map(&p.map_nope, a.kv, CU_TENSOR_MAP_DATA_TYPE_UINT8, M1_DATA_BYTES, vrows, M1_DATA_BYTES, 256, CU_TENSOR_MAP_SWIZZLE_NONE)) return rc;
    if (int rc = tc::make_row_map(&p.map_rope, a.kv, CU_TENSOR_MAP_DATA_TYPE_UINT8, M1_DATA_BYTES, vrows, M1_DATA_BYTES, 192, CU_TENSOR_MAP_SWIZZLE_NONE)) return rc;
    if (int rc = tc::make_row_map(&p.map_scale, a.kv, CU_TENSOR_MAP_DATA_TYPE_UINT8, M1_DATA_BYTES, vrows, M1_DATA_BYTES, 128, CU_TENSOR_MAP_SWIZZLE_NONE)) return rc;
    p.map_nope2 = p.map_nope; p.map_rope2 = p.map_rope; p.map_scale2 = p.map_scale;      // replaced below when there is an extra cache
    if (a.extra_kv != nullptr) {
      p.rows_per_block2 = (int)(a.extra_kv_stride_block / M1_DATA_BYTES);
      const uint64_t vrows2 = (uint64_t)(a.extra_num_blocks - 1) * p.rows_per_block2 + a.extra_page_block_size;
      if (int rc = tc::make_row_map(&p.map_nope2, a.extra_kv, CU_TENSOR_MAP_DATA_TYPE_UINT8, M1_DATA_BYTES, vrows2, M1_DATA_BYTES, 256, CU_TENSOR_MAP_SWIZZLE_NONE)) return rc;
      if (int rc = tc::make_row_map(&p.map_rope2, a.extra_kv, CU_TENSOR_MAP_DATA_TYPE_UINT8, M1_DATA_BYTES, vrows2, M1_DATA_BYTES, 192, CU_TENSOR_MAP_SWIZZLE_NONE)) return rc;
      if (int rc = tc::make_row_map(&p.map_scale2, a.extra_kv, CU_TENSOR_MAP_DATA_TYPE_UINT8, M1_DATA_BYTES, vrows2, M1_DATA_BYTES, 128, CU_TENSOR_MAP_SWIZZLE_NONE)) return rc;
      p.has_extra = 1;
      p.kv_rows2 = reinterpret_cast<const uint8_t*>(a.extra_kv);
      p.kv_stride_block2 = a.extra_kv_stride_block;
      p.page2 = (int)a.extra_page_block_size;
      p.total_rows2 = a.extra_num_blocks * a.extra_page_block_size;
      p.extra_topk = a.extra_topk;
      p.extra_topk_length = a.extra_topk_length;
      p.indices2 = a.extra_indices; p.idx2_stride0 = a.extra_idx_stride_b; p.idx2_stride1 = a.extra_idx_stride_s;
    }
    return tc::launch(p, dim3(2 * a.num_sm_parts, a.s_q, (a.h_q + 127) / 128), stream);
  }
  p.rows_per_block = (int)(a.kv_stride_block / ROW_BYTES);
  const uint64_t vrows = (uint64_t)(a.num_blocks - 1) * p.rows_per_block + a.page_block_size;
  if (int rc = tc::make_row_map(&p.map_nope, a.kv, CU_TENSOR_MAP_DATA_TYPE_UINT8, ROW_BYTES, vrows, ROW_BYTES, 256, CU_TENSOR_MAP_SWIZZLE_NONE)) return rc;
  if (int rc = tc::make_row_map(&p.map_rope, a.kv, CU_TENSOR_MAP_DATA_TYPE_UINT8, ROW_BYTES, vrows, ROW_BYTES, 64, CU_TENSOR_MAP_SWIZZLE_NONE)) return rc;
  if (int rc = tc::make_row_map(&p.map_scale, a.kv, CU_TENSOR_MAP_DATA_TYPE_UINT8, ROW_BYTES, vrows, ROW_BYTES, 16, CU_TENSOR_MAP_SWIZZLE_NONE)) return rc;
  p.map_nope2 = p.map_nope; p.map_rope2 = p.map_rope; p.map_scale2 = p.map_scale;      // replaced below when there is an extra cache
  if (a.extra_kv != nullptr) {
    const uint64_t vrows2 = (uint64_t)(a.extra_num_blocks - 1) * (uint64_t)(a.extra_kv_stride_block / ROW_BYTES) + a.extra_page_block_size;
    if (int rc = tc::make_row_map(&p.map_nope2, a.extra_kv, CU_TENSOR_MAP_DATA_TYPE_UINT8, ROW_BYTES, vrows2, ROW_BYTES, 256, CU_TENSOR_MAP_SWIZZLE_NONE)) return rc;
    if (int rc = tc::make_row_map(&p.map_rope2, a.extra_kv, CU_TENSOR_MAP_DATA_TYPE_UINT8, ROW_BYTES, vrows2, ROW_BYTES, 64, CU_TENSOR_MAP_SWIZZLE_NONE)) return rc;
    if (int rc = tc::make_row_map(&p.map_scale2, a.extra_kv, CU_TENSOR_MAP_DATA_TYPE_UINT8, ROW_BYTES, vrows2, ROW_BYTES, 16, CU_TENSOR_MAP_SWIZZLE_NONE)) return rc;
    p.has_extra = 1;
    p.kv_rows2 = reinterpret_cast<const uint8_t*>(a.extra_kv);
    p.rows_per_block2 = (int)(a.extra_kv_stride_block / ROW_BYTES);
    p.page2 = (int)a.extra_page_block_size;
    p.total_rows2 = a.extra_num_blocks * a.extra_page_block_size;
    p.extra_topk = a.extra_topk;
    p.extra_topk_length = a.extra_topk_length;
    p.indices2 = a.extra_indices; p.idx2_stride0 = a.extra_idx_stride_b; p.idx2_stride1 = a.extra_idx_stride_s;
  }
  return tc::launch(p, dim3(2 * a.num_sm_parts, a.s_q, (a.h_q + 127) / 128), stream);
}

int launch_tc_dense_decode(const FmlaDenseDecodeArgs& a, cudaStream_t stream) {
  tc::Params p = {};
  p.mode = 0;
  p.d_qk = D_QK;
  p.h_q = a.h_q;
  p.topk = (int)(a.max_blocks_per_seq * a.page_block_size);     // the longest token list a block table row can describe
  p.scale_log2 = a.sm_scale * LOG2E;
  p.q = reinterpret_cast<const __nv_bfloat16*>(a.q);
  p.q_stride0 = a.q_stride_b; p.q_stride1 = a.q_stride_s; p.q_stride_h = a.q_stride_h;
  p.q_tma = tc::make_q_map(&p.map_q, a.q, a.h_q, (uint64_t)a.s_q, (uint64_t)a.b, a.q_stride_h, a.q_stride_s, a.q_stride_b, 64, CU_TENSOR_MAP_SWIZZLE_128B, D_QK) &&
            tc::make_q_map(&p.map_q_rope, a.q, a.h_q, (uint64_t)a.s_q, (uint64_t)a.b, a.q_stride_h, a.q_stride_s, a.q_stride_b, 32, CU_TENSOR_MAP_SWIZZLE_64B, D_QK);
  p.block_table = a.block_table; p.block_table_stride = a.block_table_stride;
  p.topk_length = a.cache_seqlens;
  p.causal = a.causal && a.s_q > 1;
  p.page = (int)a.page_block_size;
  p.kv_bf16 = reinterpret_cast<const __nv_bfloat16*>(a.kv);
  p.kv_stride_s = a.kv_stride_row;
  p.s_kv = (int)(a.num_blocks * a.page_block_size);
  p.dense_blocks = (int)a.num_blocks;
  p.sched = reinterpret_cast<const SchedRecord*>(a.sched_meta); p.num_splits = a.num_splits;
  p.b = a.b; p.s_q = a.s_q;
  p.out = reinterpret_cast<__nv_bfloat16*>(a.out);
  p.o_stride0 = a.o_stride_b; p.o_stride1 = a.o_stride_s; p.o_stride_h = a.o_stride_h;
  p.lse = a.lse; p.lse_stride0 = a.lse_stride_b; p.lse_stride1 = a.lse_stride_s;
  p.o_accum = a.o_accum; p.lse_accum = a.lse_accum;
  p.status = a.status;
  const uint64_t acc_rows = (uint64_t)(a.b + a.num_sm_parts) * (uint64_t)a.s_q;
  p.out_tma = tc::make_out_map(&p.map_out, a.out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.h_q, (uint64_t)a.s_q, (uint64_t)a.b, a.o_stride_h, a.o_stride_s, a.o_stride_b, 32) &&
              tc::make_out_map(&p.map_acc, a.o_accum, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a.h_q, acc_rows, 1, D_V, (int64_t)a.h_q * D_V, (int64_t)(acc_rows * a.h_q) * D_V, 16);
  if (int rc = tc::make_row_map(&p.map_nope, a.kv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, D_QK, (uint64_t)p.s_kv, (uint64_t)a.kv_stride_row * 2, 64, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  if (int rc = tc::make_row_map(&p.map_rope, a.kv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, D_QK, (uint64_t)p.s_kv, (uint64_t)a.kv_stride_row * 2, 32, CU_TENSOR_MAP_SWIZZLE_64B)) return rc;
  return tc::launch(p, dim3(2 * a.num_sm_parts, a.s_q, (a.h_q + 127) / 128), stream);
}

int launch_tc_prefill_fwd(const FmlaPrefillArgs& a, cudaStream_t stream) {
  tc::Params p = {};
  p.mode = 1;
  p.h_q = a.h_q; p.topk = a.topk;
  FMLA_REQUIRE(a.sm_scale > 0.f, FMLA_ERR_UNSUPPORTED, "the tensor-core kernel needs a positive softmax scale (got %g); use FMLA_KERNEL_SIMT", (double)a.sm_scale);
  p.scale_log2 = a.sm_scale * LOG2E;
  p.q = reinterpret_cast<const __nv_bfloat16*>(a.q);
  p.q_stride0 = a.q_stride_s; p.q_stride1 = 0; p.q_stride_h = a.q_stride_h;
  // d_qk = 512: q and kv rows hold 512 values and V is all of them.  The maps are made over 512 columns and the TMA
  // unit zero-fills what lies beyond, so the kernel sees 576-wide rows whose last 64 features are zero: the first 512
  // features of a row are V either way, and zero features add nothing to q . k.
  const int d_qk = a.d_qk == 0 ? D_QK : a.d_qk;
  p.d_qk = d_qk;
  p.q_tma = tc::make_q_map(&p.map_q, a.q, a.h_q, (uint64_t)a.s_q, 1, a.q_stride_h, a.q_stride_s, a.q_stride_s * a.s_q, 64, CU_TENSOR_MAP_SWIZZLE_128B, d_qk) &&
            tc::make_q_map(&p.map_q_rope, a.q, a.h_q, (uint64_t)a.s_q, 1, a.q_stride_h, a.q_stride_s, a.q_stride_s * a.s_q, 32, CU_TENSOR_MAP_SWIZZLE_64B, d_qk);
  p.indices = a.indices; p.idx_stride0 = a.idx_stride_s; p.idx_stride1 = 0;
  p.topk_length = a.topk_length; p.attn_sink = a.attn_sink;
  p.kv_bf16 = reinterpret_cast<const __nv_bfloat16*>(a.kv);
  p.kv_stride_s = a.kv_stride_s; p.s_kv = a.s_kv; p.n_queries = a.s_q;
  p.out = reinterpret_cast<__nv_bfloat16*>(a.out);
  p.lse = a.lse; p.max_logits = a.max_logits;
  p.status = a.status;
  p.out_tma = tc::make_out_map(&p.map_out, a.out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.h_q, (uint64_t)a.s_q, 1, D_V, (int64_t)a.h_q * D_V, (int64_t)a.h_q * D_V * a.s_q, 32);
  if (int rc = tc::make_row_map(&p.map_nope, a.kv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, d_qk, (uint64_t)a.s_kv, (uint64_t)a.kv_stride_s * 2, 64, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  if (int rc = tc::make_row_map(&p.map_rope, a.kv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, d_qk, (uint64_t)a.s_kv, (uint64_t)a.kv_stride_s * 2, 32, CU_TENSOR_MAP_SWIZZLE_64B)) return rc;
  const int groups = (a.h_q + 127) / 128;
  int clusters = sm_count() / 2 / groups;
  if (clusters < 1) clusters = 1;
  if (clusters > a.s_q) clusters = a.s_q;
  return tc::launch(p, dim3(2 * clusters, 1, groups), stream);
}

}  // namespace fmla
