/*
 * flashmla_b200 — C ABI of the B200 (sm_100a) token-level sparse MLA attention library.
 *
 * Every entry point takes plain pointers and sizes, enqueues work on the given CUDA stream
 * and returns immediately (no stream synchronisation, no device allocation, no frees).
 * All device buffers — inputs, outputs, scheduler metadata and split-KV scratch — are owned
 * by the caller and must stay valid until the enqueued work has run; the one exception is
 * fmla_sparse_decode_static_scratch, whose split-KV scratch is an array inside the library.  Return value 0 means
 * success; any other value is one of the FMLA_ERR_* codes and fmla_last_error() returns a
 * thread-local, human readable description.  Nothing here calls exit() or traps the device.
 *
 * Each declaration cites the interface of the reference implementation that it replaces
 * (paths are relative to the reference project's root).
 */
#ifndef FLASHMLA_B200_H_
#define FLASHMLA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FMLA_OK               0
#define FMLA_ERR_INVALID_ARG  1   /* null pointer, bad shape, negative size */
#define FMLA_ERR_UNSUPPORTED  2   /* shape / layout combination no kernel covers */
#define FMLA_ERR_ALIGNMENT    3   /* base pointer or stride not aligned as the kernels require */
#define FMLA_ERR_CUDA         4   /* a CUDA runtime call failed; message carries cudaGetErrorString */
#define FMLA_ERR_ARCH         5   /* device is not compute capability 10.x */
#define FMLA_ERR_TIMEOUT      6   /* a bounded device-side wait gave up (reported through a status word) */

/*
 * Values of the optional device status word (FmlaDecodeArgs.status and its siblings), which starts at 0 and keeps the
 * first non-zero value written to it:
 *   1 .. 99             a kernel gave up a bounded wait (the number names the wait); the call's results are invalid.
 *   FMLA_STATUS_CLIPPED  the tensor-core decode kernel stages the dequantised NoPE part and Q in fp16 and met a value
 *                       outside that range: a cache scale above 2^7 (a row whose tile maximum exceeds 57344) or a
 *                       |q| above 65504.  Such values were clipped, so the call's results are not to be trusted; run
 *                       the call again with FMLA_KERNEL_SIMT, which multiplies in fp32 like the reference
 *                       (tests/quant.py:93-104).  FMLA_KERNEL_AUTO cannot know the values in advance and picks the
 *                       tensor-core kernel whenever the shape allows.
 */
#define FMLA_STATUS_CLIPPED 100

/* KV-cache layouts, one KV head.  V32 and MXFP8: 656 bytes per token, d_qk = 576 (512 NoPE + 64 RoPE). */
#define FMLA_LAYOUT_V32    0   /* 512 e4m3 | 4 x fp32 scale (per 128) | 64 bf16   (flash_mla/flash_mla_interface.py:94-98) */
#define FMLA_LAYOUT_MXFP8  1   /* 512 e4m3 | 16 x e8m0 scale (per 32) | 64 bf16   (no counterpart in the reference) */
/* MODEL1: d_qk = 512 (448 NoPE + 64 RoPE), 584 bytes per token, stored per cache block as
 * [page_block_size x (448 e4m3 | 64 bf16)] followed by [page_block_size x (7 e8m0 scales, one per 64 values, | 1 pad byte)]
 * (tests/quant.py:55-75 of the reference; its decode dispatches on d_qk, csrc/api/sparse_decode.h:318-325).  The
 * value dimension is still 512: the RoPE part belongs to V. */
#define FMLA_LAYOUT_MODEL1 2
#define FMLA_MODEL1_ROW_BYTES   584
#define FMLA_MODEL1_DATA_BYTES  576   /* the part of a token's bytes that sits in the block's leading array */
#define FMLA_MODEL1_D_QK        512

#define FMLA_D_QK        576
#define FMLA_D_V         512
#define FMLA_ROW_BYTES   656
#define FMLA_STATIC_SCRATCH_ROWS 16384   /* accumulator rows of fmla_sparse_decode_static_scratch's built-in array */
#define FMLA_SCHED_META_INTS 8  /* one partition record: csrc/params.h:10-17 (DecodingSchedMeta) */

/* Kernel selection for the attention entry points. */
#define FMLA_KERNEL_AUTO   0   /* tensor-core kernel when the shape allows, else the generic one */
#define FMLA_KERNEL_SIMT   1   /* generic CUDA-core kernel (any head count) */
#define FMLA_KERNEL_TC     2   /* tcgen05 kernel (h_q a multiple of 64; groups of 128 heads, a last group of 64 runs half empty) */

int fmla_version(void);
const char* fmla_last_error(void);

/*
 * Process-wide switches, for diagnosis and tests.  No counterpart in the reference.
 *   FMLA_OPTION_PLAIN_Q_LOADS  non-zero: the tensor-core attention kernel reads Q with plain loads instead of TMA
 *                              tiles (the path it otherwise takes only when the driver refuses q's strides).
 *   FMLA_OPTION_PLAIN_STORES   non-zero: the tensor-core attention kernel writes its results with plain stores instead
 *                              of TMA box stores (the path it otherwise takes only when the driver refuses out's strides).
 */
#define FMLA_OPTION_PLAIN_Q_LOADS 1
#define FMLA_OPTION_PLAIN_STORES  2
int fmla_set_option(int option, int value);

/*
 * Hits and misses of the library's table of encoded TMA descriptors.  The reference encodes its descriptors on every
 * call (csrc/sm100/decode/head64/kernel.cuh:913-930); here a call whose buffers and shapes were seen before encodes none.
 */
int fmla_tensor_map_cache_stats(uint64_t* hits, uint64_t* misses);

/*
 * Split-KV plan for a decode shape on `device`: how many SM partitions the decode kernel is
 * launched with, the per-request fixed overhead (in token blocks) the scheduler assumes, and the
 * token block size.  Replaces DecodeImplBase::get_meta (csrc/api/sparse_decode.h:30-34,92-99,168-175).
 */
int fmla_decode_plan(int device, int h_q, int s_q, int kernel,
                     int* num_sm_parts, int* fixed_overhead_blocks, int* block_topk);

/*
 * Tile scheduler: partitions the token blocks of all requests over num_sm_parts partitions.
 * Writes sched_meta [num_sm_parts][8] int32 and num_splits [b+1] int32 (both device pointers).
 * topk_length may be null (every request uses `topk`).  Replaces run_get_decoding_sched_meta_kernel
 * (csrc/smxx/decode/get_decoding_sched_meta/get_decoding_sched_meta.cu:11-114) for the sparse case.
 */
typedef struct {
  int device;
  int b, topk;
  int block_topk, fixed_overhead_blocks, num_sm_parts;
  const int32_t* topk_length;   /* [b] or null */
  int32_t* sched_meta;          /* [num_sm_parts, 8] */
  int32_t* num_splits;          /* [b+1] */
  int extra_topk;               /* 0, or the width of the extra index list (see FmlaDecodeArgs.extra_kv) */
  const int32_t* extra_topk_length;   /* [b] or null */
} FmlaSchedArgs;
int fmla_sched_meta(const FmlaSchedArgs* args, void* cuda_stream);

/*
 * Sparse decode over a paged FP8 / MXFP8 KV cache: split-KV attention kernel followed by the combine
 * kernel.  Replaces sparse_attn_decode_interface (csrc/api/sparse_decode.h:183-495; Python binding
 * flash_mla_cuda.sparse_decode_fwd, csrc/api/api.cpp:10) minus its allocations: out, lse, the
 * scheduler outputs (filled by fmla_sched_meta beforehand) and the two accumulators are passed in.
 * Strides are in elements of the pointed-to type, except the KV strides which are in bytes.
 */
typedef struct {
  int device;
  int b, s_q, h_q, topk;
  int layout;                    /* FMLA_LAYOUT_* */
  int kernel;                    /* FMLA_KERNEL_* */
  float sm_scale;
  const void* q;                 /* bf16 [b, s_q, h_q, 576] (512 with FMLA_LAYOUT_MODEL1), last dim contiguous */
  int64_t q_stride_b, q_stride_s, q_stride_h;
  const void* kv;                /* bytes [num_blocks, page_block_size, 656] (MODEL1: blocks as described at FMLA_LAYOUT_MODEL1) */
  int64_t num_blocks, page_block_size;
  int64_t kv_stride_block;       /* bytes, multiple of 16 */
  const int32_t* indices;        /* [b, s_q, topk]: block*page_block_size + offset, or -1 */
  int64_t idx_stride_b, idx_stride_s;
  const int32_t* topk_length;    /* [b] or null */
  const float* attn_sink;        /* [h_q] or null */
  void* out;                     /* bf16 [b, s_q, h_q, 512] */
  int64_t o_stride_b, o_stride_s, o_stride_h;
  float* lse;                    /* fp32 [b, s_q, h_q], natural log */
  int64_t lse_stride_b, lse_stride_s;
  const int32_t* sched_meta;     /* [num_sm_parts, 8] from fmla_sched_meta */
  const int32_t* num_splits;     /* [b+1] */
  int num_sm_parts;
  float* o_accum;                /* fp32 [b + num_sm_parts, s_q, h_q, 512] scratch */
  float* lse_accum;              /* fp32 [b + num_sm_parts, s_q, h_q] scratch */
  int32_t* status;               /* optional device word; a kernel that gave up a bounded wait sets it non-zero */
  void* attn_done_event;         /* optional cudaEvent_t recorded on the stream between the attention and the combine
                                    kernel, so that a caller can time the two separately; null = not recorded */
  /* Optional second cache (extra_k_cache of flash_mla_with_kvcache, flash_mla_interface.py:66-69,88-90): every query
     also attends to extra_indices' rows of extra_kv.  A request's token list is its first topk_length (or topk)
     main slots, padded to a multiple of 64, followed by its first extra_topk_length (or extra_topk) extra slots
     (get_decoding_sched_meta.cu:37-42); the scheduler output must have been made with the same extra fields. */
  const void* extra_kv;          /* bytes [extra_num_blocks, extra_page_block_size, 656] in the same layout, or null */
  int64_t extra_num_blocks, extra_page_block_size, extra_kv_stride_block;
  const int32_t* extra_indices;  /* [b, s_q, extra_topk] */
  int64_t extra_idx_stride_b, extra_idx_stride_s;
  int extra_topk;
  const int32_t* extra_topk_length;   /* [b] or null */
} FmlaDecodeArgs;
int fmla_sparse_decode(const FmlaDecodeArgs* args, void* cuda_stream);

/*
 * fmla_sparse_decode without caller-provided accumulators.  No counterpart in the reference, whose
 * interface allocates its accumulators with torch on every call (csrc/api/sparse_decode.h).
 * args->o_accum and args->lse_accum must be null; the split-KV partial results go to a fixed array
 * (32 MiB + 64 KiB) inside the library's device image, and the call allocates nothing.
 *   limit     (b + num_sm_parts) * s_q * h_q <= FMLA_STATIC_SCRATCH_ROWS, else FMLA_ERR_UNSUPPORTED.
 *   set-up    the first call on a device looks the array's address up (which may load the module on that
 *             device); make that call before any stream capture.  Later calls only launch the two kernels.
 *             The address is kept for the life of the process: after a cudaDeviceReset of that device (which
 *             unloads the module) it is stale and this entry point must not be used on it again.
 *   sharing   one array per device: calls on one device that may overlap in time (different streams
 *             or host threads) race on it, so order them on one stream or by events.  The array keeps the
 *             last call's contents; nothing in it needs clearing between calls.
 * Everything else (validation, kernels, results) is fmla_sparse_decode's.
 */
int fmla_sparse_decode_static_scratch(const FmlaDecodeArgs* args, void* cuda_stream);

/*
 * Dense decode over a paged bf16 cache with one KV head: every query attends all cache_seqlens[i] tokens of its request
 * (with `causal`, query row j of s_q sees the first cache_seqlens[i] - (s_q - 1 - j)), found through the block table.
 * Split-KV attention on the tensor-core kernel followed by the combine kernel, as in fmla_sparse_decode.  Replaces
 * dense_attn_decode_interface (csrc/api/dense_decode.h:13-24; Python binding flash_mla_cuda.dense_decode_fwd), which
 * the reference builds for sm_90a only (csrc/api/dense_decode.h:27-29), minus its allocations.  The scheduler output
 * comes from fmla_sched_meta with topk = max_blocks_per_seq * page_block_size, topk_length = cache_seqlens and the
 * plan of fmla_decode_plan(device, h_q, s_q, FMLA_KERNEL_TC).  h_q must be a multiple of 64.
 * A request of length 0 (or rows that see no token) gets out = 0 and lse = +inf.  Any page_block_size works (the
 * reference takes 64 only, csrc/api/dense_decode.h:67); a block-table entry outside [0, num_blocks) makes its tokens
 * invalid slots (they contribute nothing), as -1 does in an index list.
 */
typedef struct {
  int device;
  int b, s_q, h_q;
  int causal;
  float sm_scale;                /* > 0 */
  const void* q;                 /* bf16 [b, s_q, h_q, 576], last dim contiguous */
  int64_t q_stride_b, q_stride_s, q_stride_h;
  const void* kv;                /* bf16 [num_blocks * page_block_size, 576]: the cache's rows at one pitch */
  int64_t num_blocks, page_block_size;
  int64_t kv_stride_row;         /* elements, multiple of 8 */
  const int32_t* block_table;    /* [b, max_blocks_per_seq]: cache block of each page of a request */
  int64_t block_table_stride;
  int64_t max_blocks_per_seq;
  const int32_t* cache_seqlens;  /* [b] */
  void* out;                     /* bf16 [b, s_q, h_q, 512] */
  int64_t o_stride_b, o_stride_s, o_stride_h;
  float* lse;                    /* fp32 [b, s_q, h_q], natural log */
  int64_t lse_stride_b, lse_stride_s;
  const int32_t* sched_meta;     /* [num_sm_parts, 8] */
  const int32_t* num_splits;     /* [b+1] */
  int num_sm_parts;
  float* o_accum;                /* fp32 [b + num_sm_parts, s_q, h_q, 512] scratch */
  float* lse_accum;              /* fp32 [b + num_sm_parts, s_q, h_q] scratch */
  int32_t* status;               /* optional, as in FmlaDecodeArgs */
} FmlaDenseDecodeArgs;
int fmla_dense_decode(const FmlaDenseDecodeArgs* args, void* cuda_stream);

/*
 * Sparse prefill forward.  Replaces sparse_attn_prefill_interface (csrc/api/sparse_fwd.h:101-243;
 * Python binding flash_mla_cuda.sparse_prefill_fwd, csrc/api/api.cpp:12); outputs are passed in.
 */
typedef struct {
  int device;
  int s_q, s_kv, h_q, topk;
  int kernel;
  float sm_scale;
  const void* q;                 /* bf16 [s_q, h_q, d_qk] */
  int64_t q_stride_s, q_stride_h;
  const void* kv;                /* bf16 [s_kv, 1, d_qk] */
  int64_t kv_stride_s;           /* elements */
  const int32_t* indices;        /* [s_q, 1, topk]; valid iff 0 <= idx < s_kv */
  int64_t idx_stride_s;
  const float* attn_sink;        /* [h_q] or null */
  const int32_t* topk_length;    /* [s_q] or null */
  void* out;                     /* bf16 [s_q, h_q, 512] contiguous */
  float* max_logits;             /* fp32 [s_q, h_q] */
  float* lse;                    /* fp32 [s_q, h_q] */
  int32_t* status;               /* optional, as in FmlaDecodeArgs */
  int d_qk;                      /* 576, or 512 (q and kv rows of 512 values; the reference's d_qk = 512 prefill,
                                    csrc/api/sparse_fwd.h:213-240); 0 means 576 */
} FmlaPrefillArgs;
int fmla_sparse_prefill_fwd(const FmlaPrefillArgs* args, void* cuda_stream);

/*
 * Sparse prefill backward: dq (bf16) and dkv (fp32 scatter-add over duplicate indices, then an
 * optional bf16 copy).  The reference has no sparse backward (csrc/api/api.cpp:8-15 exports none);
 * the argument meaning follows the forward entry point.  `lse` is the forward's lse output.
 * dkv_accum is zeroed by the call before accumulation.
 */
typedef struct {
  int device;
  int s_q, s_kv, h_q, topk;
  int kernel;
  float sm_scale;
  const void* q;  int64_t q_stride_s, q_stride_h;
  const void* kv; int64_t kv_stride_s;
  const void* out;               /* bf16 [s_q, h_q, 512] contiguous (forward output) */
  const void* dout;              /* bf16 [s_q, h_q, 512] */
  int64_t do_stride_s, do_stride_h;
  const float* lse;              /* fp32 [s_q, h_q] */
  const int32_t* indices; int64_t idx_stride_s;
  const float* attn_sink;        /* or null */
  const int32_t* topk_length;    /* or null */
  void* dq;                      /* bf16 [s_q, h_q, 576] contiguous */
  float* dkv_accum;              /* fp32 [s_kv, 576] contiguous */
  void* dkv;                     /* bf16 [s_kv, 576] contiguous, or null to skip the cast */
  void* workspace;               /* tensor-core kernels only: 128-byte aligned scratch for P and dS in bf16; any size
                                    >= fmla_sparse_prefill_bwd_workspace(1, h_q, topk) works, the query tokens are
                                    processed in as many chunks as the size makes necessary */
  int64_t workspace_bytes;
  int32_t* status;               /* optional, as in FmlaDecodeArgs */
  void* grad_begin_event;        /* optional cudaEvent_t pair recorded on the stream around the first pass's dQ / dKV */
  void* grad_end_event;          /* launch (tensor-core kernels), so that a caller can time that launch; null = not recorded */
} FmlaPrefillBwdArgs;
int fmla_sparse_prefill_bwd(const FmlaPrefillBwdArgs* args, void* cuda_stream);
/* Workspace bytes with which `s_q` query tokens go through the tensor-core backward in one chunk (0 when the
 * head count runs on the CUDA-core kernels, which need none).  kernel = FMLA_KERNEL_AUTO / _TC / _SIMT. */
int64_t fmla_sparse_prefill_bwd_workspace(int s_q, int h_q, int topk, int kernel);

/*
 * KV-cache writer: quantises bf16 rows [576] into 656-byte cache rows of the given layout (FMLA_LAYOUT_MODEL1: rows
 * [512] into the block-wise 584-byte form, with rows_stride_block >= page_block_size * 584).  Replaces the torch
 * fixture quantize_k_cache (tests/quant.py:20-78; the reference ships no kernel for it) byte for byte for the V32
 * layout; the MXFP8 layout applies the same scale rule per 32 values.  Row i goes to
 * rows + (i / page_block_size) * rows_stride_block + (i % page_block_size) * 656.
 */
typedef struct {
  int device;
  int layout;                    /* FMLA_LAYOUT_* */
  int64_t n_rows, page_block_size;
  const void* kv;                /* bf16 [n_rows, 576], last dim contiguous, 16-byte aligned */
  int64_t kv_stride_row;         /* elements, multiple of 8 */
  void* rows;                    /* bytes, 16-byte aligned */
  int64_t rows_stride_block;     /* bytes, multiple of 16, >= page_block_size * 656 */
} FmlaKvQuantArgs;
int fmla_kv_quantize(const FmlaKvQuantArgs* args, void* cuda_stream);

/*
 * Logical token positions -> in-cache row indices through the block table; replaces the torch helper
 * abs_indices2indices_in_kvcache (tests/quant.py:126-158):
 * indices[i, j] = block_table[i, p / page] * page + p % page for p = positions[i, j] >= 0, else -1.
 */
typedef struct {
  int device;
  int b, page_block_size, max_pages;
  int64_t per_request;           /* positions per request (s_q * topk), contiguous */
  const int32_t* positions;      /* [b, per_request] */
  const int32_t* block_table;    /* [b, max_pages] */
  int32_t* indices;              /* [b, per_request] */
} FmlaCacheIndexArgs;
int fmla_cache_indices(const FmlaCacheIndexArgs* args, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif  /* FLASHMLA_B200_H_ */
