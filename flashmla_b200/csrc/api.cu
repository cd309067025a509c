// C ABI of flashmla_b200: argument validation, kernel selection and launch sequencing.
// Validation is pure host code and runs before any CUDA call, so bad arguments are reported
// identically with or without a GPU.
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace fmla {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

namespace {

struct DeviceInfo {
  bool known = false;
  int major = 0, minor = 0, sms = 0;
};
constexpr int MAX_DEVICES = 64;
DeviceInfo g_devices[MAX_DEVICES];
std::mutex g_devices_mu;

int device_info(int device, DeviceInfo* out) {
  FMLA_REQUIRE(device >= 0 && device < MAX_DEVICES, FMLA_ERR_INVALID_ARG, "device ordinal %d out of range", device);
  std::lock_guard<std::mutex> lock(g_devices_mu);
  DeviceInfo& d = g_devices[device];
  if (!d.known) {
    FMLA_CUDA(cudaDeviceGetAttribute(&d.major, cudaDevAttrComputeCapabilityMajor, device));
    FMLA_CUDA(cudaDeviceGetAttribute(&d.minor, cudaDevAttrComputeCapabilityMinor, device));
    FMLA_CUDA(cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, device));
    d.known = true;
  }
  *out = d;
  FMLA_REQUIRE(d.major == 10, FMLA_ERR_ARCH,
               "device %d has compute capability %d.%d; these kernels are built for sm_100a only", device, d.major,
               d.minor);
  return FMLA_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int pick_kernel(int requested, int h_q, const char* what) {
  if (requested == FMLA_KERNEL_SIMT) return FMLA_KERNEL_SIMT;
  const bool tc_ok = tc_supported(h_q);
  if (requested == FMLA_KERNEL_TC) {
    if (!tc_ok) {
      set_error("%s: the tensor-core kernel needs h_q to be a multiple of 64 (got %d)", what, h_q);
      return -1;
    }
    return FMLA_KERNEL_TC;
  }
  return tc_ok ? FMLA_KERNEL_TC : FMLA_KERNEL_SIMT;
}

}  // namespace
}  // namespace fmla

using namespace fmla;

extern "C" {

int fmla_version(void) { return 132; }   // 130: fmla_set_option, fmla_tensor_map_cache_stats, FMLA_STATUS_* codes; 131: FMLA_OPTION_PLAIN_STORES, MODEL1 on the tensor cores; 132: fmla_dense_decode

const char* fmla_last_error(void) { return g_error; }

int fmla_decode_plan(int device, int h_q, int s_q, int kernel, int* num_sm_parts, int* fixed_overhead_blocks,
                     int* block_topk) {
  FMLA_REQUIRE(num_sm_parts && fixed_overhead_blocks && block_topk, FMLA_ERR_INVALID_ARG, "decode_plan: null output pointer");
  FMLA_REQUIRE(h_q > 0 && s_q > 0, FMLA_ERR_INVALID_ARG, "decode_plan: h_q=%d s_q=%d must be positive", h_q, s_q);
  const int k = pick_kernel(kernel, h_q, "decode_plan");
  if (k < 0) return FMLA_ERR_UNSUPPORTED;
  DeviceInfo info;
  if (int rc = device_info(device, &info)) return rc;
  if (k == FMLA_KERNEL_TC) return tc_decode_plan(info.sms, h_q, s_q, num_sm_parts, fixed_overhead_blocks, block_topk);
  // Generic kernel: one block per (partition, query token, 16 heads), three blocks resident per SM.
  const int blocks_per_part = s_q * ((h_q + 15) / 16);
  int parts = (info.sms * 3 + blocks_per_part - 1) / blocks_per_part;
  parts = parts < 1 ? 1 : (parts > 4 * info.sms ? 4 * info.sms : parts);
  *num_sm_parts = parts;
  *fixed_overhead_blocks = 5;
  *block_topk = 64;
  return FMLA_OK;
}

int fmla_sched_meta(const FmlaSchedArgs* a, void* cuda_stream) {
  FMLA_REQUIRE(a != nullptr, FMLA_ERR_INVALID_ARG, "sched_meta: null argument struct");
  FMLA_REQUIRE(a->b > 0 && a->topk > 0, FMLA_ERR_INVALID_ARG, "sched_meta: b=%d topk=%d must be positive", a->b, a->topk);
  FMLA_REQUIRE(a->block_topk > 0 && a->fixed_overhead_blocks >= 0 && a->num_sm_parts > 0, FMLA_ERR_INVALID_ARG,
               "sched_meta: block_topk=%d overhead=%d num_sm_parts=%d invalid", a->block_topk, a->fixed_overhead_blocks,
               a->num_sm_parts);
  FMLA_REQUIRE(a->extra_topk >= 0, FMLA_ERR_INVALID_ARG, "sched_meta: extra_topk=%d must not be negative", a->extra_topk);
  FMLA_REQUIRE(a->sched_meta && a->num_splits, FMLA_ERR_INVALID_ARG, "sched_meta: null output pointer");
  FMLA_REQUIRE((reinterpret_cast<uintptr_t>(a->sched_meta) & 31u) == 0, FMLA_ERR_ALIGNMENT,
               "sched_meta: metadata buffer must be 32-byte aligned");
  DeviceInfo info;
  if (int rc = device_info(a->device, &info)) return rc;
  DeviceGuard guard(a->device);
  FMLA_REQUIRE(guard.ok, FMLA_ERR_CUDA, "sched_meta: cannot switch to device %d", a->device);
  return launch_sched_meta(*a, static_cast<cudaStream_t>(cuda_stream));
}

int fmla_sparse_decode(const FmlaDecodeArgs* a, void* cuda_stream) {
  FMLA_REQUIRE(a != nullptr, FMLA_ERR_INVALID_ARG, "sparse_decode: null argument struct");
  FMLA_REQUIRE(a->b > 0 && a->s_q > 0 && a->h_q > 0 && a->topk > 0, FMLA_ERR_INVALID_ARG,
               "sparse_decode: b=%d s_q=%d h_q=%d topk=%d must be positive", a->b, a->s_q, a->h_q, a->topk);
  FMLA_REQUIRE(a->layout == FMLA_LAYOUT_V32 || a->layout == FMLA_LAYOUT_MXFP8 || a->layout == FMLA_LAYOUT_MODEL1, FMLA_ERR_UNSUPPORTED,
               "sparse_decode: unknown KV layout %d", a->layout);
  const int64_t row_bytes = a->layout == FMLA_LAYOUT_MODEL1 ? FMLA_MODEL1_ROW_BYTES : FMLA_ROW_BYTES;
  FMLA_REQUIRE(a->q && a->kv && a->indices && a->out && a->lse, FMLA_ERR_INVALID_ARG,
               "sparse_decode: q, kv, indices, out and lse must be non-null");
  FMLA_REQUIRE(a->sched_meta && a->num_splits && a->o_accum && a->lse_accum && a->num_sm_parts > 0, FMLA_ERR_INVALID_ARG,
               "sparse_decode: scheduler metadata and split-KV accumulators must be provided");
  FMLA_REQUIRE(a->num_blocks > 0 && a->page_block_size > 0, FMLA_ERR_INVALID_ARG,
               "sparse_decode: num_blocks=%lld page_block_size=%lld must be positive", (long long)a->num_blocks,
               (long long)a->page_block_size);
  FMLA_REQUIRE(a->num_blocks * a->page_block_size <= 0x7fffffffLL, FMLA_ERR_UNSUPPORTED,
               "sparse_decode: the cache holds more rows than an int32 index can address");
  FMLA_REQUIRE(a->kv_stride_block >= a->page_block_size * row_bytes, FMLA_ERR_INVALID_ARG,
               "sparse_decode: kv block stride %lld is smaller than page_block_size*%lld", (long long)a->kv_stride_block, (long long)row_bytes);
  // MODEL1 blocks hold their data rows at a pitch of 576 bytes, so 16-byte row alignment needs a block stride that is a
  // multiple of 16 as well (the reference pads its blocks to a multiple of 576, tests/quant.py:57-58)
  FMLA_REQUIRE(aligned16(a->kv) && a->kv_stride_block % 16 == 0, FMLA_ERR_ALIGNMENT,
               "sparse_decode: kv base and block stride must be multiples of 16 bytes");
  FMLA_REQUIRE(aligned16(a->q) && a->q_stride_b % 8 == 0 && a->q_stride_s % 8 == 0 && a->q_stride_h % 8 == 0,
               FMLA_ERR_ALIGNMENT, "sparse_decode: q base and strides must be multiples of 16 bytes");
  FMLA_REQUIRE(aligned16(a->out) && a->o_stride_b % 8 == 0 && a->o_stride_s % 8 == 0 && a->o_stride_h % 8 == 0,
               FMLA_ERR_ALIGNMENT, "sparse_decode: out base and strides must be multiples of 16 bytes");
  FMLA_REQUIRE(aligned16(a->o_accum), FMLA_ERR_ALIGNMENT, "sparse_decode: o_accum must be 16-byte aligned");
  FMLA_REQUIRE((reinterpret_cast<uintptr_t>(a->sched_meta) & 31u) == 0, FMLA_ERR_ALIGNMENT,
               "sparse_decode: scheduler metadata must be 32-byte aligned");
  if (a->extra_kv != nullptr) {
    FMLA_REQUIRE(a->extra_indices != nullptr && a->extra_topk > 0, FMLA_ERR_INVALID_ARG,
                 "sparse_decode: extra_indices_in_kvcache must be provided when extra_k_cache is provided");
    FMLA_REQUIRE(a->extra_num_blocks > 0 && a->extra_page_block_size > 0 &&
                     a->extra_num_blocks * a->extra_page_block_size <= 0x7fffffffLL, FMLA_ERR_INVALID_ARG,
                 "sparse_decode: extra cache of %lld blocks x %lld rows is empty or holds more rows than an int32 index can address",
                 (long long)a->extra_num_blocks, (long long)a->extra_page_block_size);
    FMLA_REQUIRE(a->extra_kv_stride_block >= a->extra_page_block_size * row_bytes, FMLA_ERR_INVALID_ARG,
                 "sparse_decode: extra kv block stride %lld is smaller than page_block_size*%lld", (long long)a->extra_kv_stride_block, (long long)row_bytes);
    FMLA_REQUIRE(aligned16(a->extra_kv) && a->extra_kv_stride_block % 16 == 0, FMLA_ERR_ALIGNMENT,
                 "sparse_decode: extra kv base and block stride must be multiples of 16 bytes");
  } else {
    FMLA_REQUIRE(a->extra_indices == nullptr && a->extra_topk_length == nullptr && a->extra_topk == 0, FMLA_ERR_INVALID_ARG,
                 "sparse_decode: extra_indices_in_kvcache and extra_topk_length must not be provided when extra_k_cache is not provided");
  }
  const int k = pick_kernel(a->kernel, a->h_q, "sparse_decode");
  if (k < 0) return FMLA_ERR_UNSUPPORTED;
  DeviceInfo info;
  if (int rc = device_info(a->device, &info)) return rc;
  DeviceGuard guard(a->device);
  FMLA_REQUIRE(guard.ok, FMLA_ERR_CUDA, "sparse_decode: cannot switch to device %d", a->device);
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  // AUTO: the tensor-core kernel when the head count, the cache strides and the scale allow it, else the generic one
  // (which works with any partition count, so a plan made for the other kernel stays valid); an explicit
  // FMLA_KERNEL_TC keeps the hard error.
  const bool use_tc = k == FMLA_KERNEL_TC && (a->kernel == FMLA_KERNEL_TC || tc_decode_supported(*a));
  int rc = use_tc ? launch_tc_decode(*a, stream) : launch_simt_decode(*a, stream);
  if (rc) return rc;
  if (a->attn_done_event) FMLA_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(a->attn_done_event), stream));
  return launch_combine(*a, stream);
}

int fmla_dense_decode(const FmlaDenseDecodeArgs* a, void* cuda_stream) {
  FMLA_REQUIRE(a != nullptr, FMLA_ERR_INVALID_ARG, "dense_decode: null argument struct");
  FMLA_REQUIRE(a->b > 0 && a->s_q > 0 && a->h_q > 0, FMLA_ERR_INVALID_ARG, "dense_decode: b=%d s_q=%d h_q=%d must be positive", a->b, a->s_q, a->h_q);
  FMLA_REQUIRE(a->q && a->kv && a->block_table && a->cache_seqlens && a->out && a->lse, FMLA_ERR_INVALID_ARG,
               "dense_decode: q, kv, block_table, cache_seqlens, out and lse must be non-null");
  FMLA_REQUIRE(a->sched_meta && a->num_splits && a->o_accum && a->lse_accum && a->num_sm_parts > 0, FMLA_ERR_INVALID_ARG,
               "dense_decode: scheduler metadata and split-KV accumulators must be provided");
  FMLA_REQUIRE(a->num_blocks > 0 && a->page_block_size > 0 && a->max_blocks_per_seq > 0, FMLA_ERR_INVALID_ARG,
               "dense_decode: num_blocks=%lld page_block_size=%lld max_blocks_per_seq=%lld must be positive", (long long)a->num_blocks,
               (long long)a->page_block_size, (long long)a->max_blocks_per_seq);
  FMLA_REQUIRE(a->num_blocks * a->page_block_size <= 0x7fffffffLL && a->max_blocks_per_seq * a->page_block_size <= 0x7fffffffLL - 64, FMLA_ERR_UNSUPPORTED,
               "dense_decode: the cache or a block table row holds more rows than an int32 index can address");
  FMLA_REQUIRE(a->kv_stride_row >= FMLA_D_QK, FMLA_ERR_INVALID_ARG, "dense_decode: kv row stride %lld is smaller than 576", (long long)a->kv_stride_row);
  FMLA_REQUIRE(a->block_table_stride >= a->max_blocks_per_seq, FMLA_ERR_INVALID_ARG, "dense_decode: block table stride %lld is smaller than its row length %lld",
               (long long)a->block_table_stride, (long long)a->max_blocks_per_seq);
  FMLA_REQUIRE(aligned16(a->kv) && a->kv_stride_row % 8 == 0, FMLA_ERR_ALIGNMENT, "dense_decode: kv base and row stride must be multiples of 16 bytes");
  FMLA_REQUIRE(aligned16(a->q) && a->q_stride_b % 8 == 0 && a->q_stride_s % 8 == 0 && a->q_stride_h % 8 == 0,
               FMLA_ERR_ALIGNMENT, "dense_decode: q base and strides must be multiples of 16 bytes");
  FMLA_REQUIRE(aligned16(a->out) && a->o_stride_b % 8 == 0 && a->o_stride_s % 8 == 0 && a->o_stride_h % 8 == 0,
               FMLA_ERR_ALIGNMENT, "dense_decode: out base and strides must be multiples of 16 bytes");
  FMLA_REQUIRE(aligned16(a->o_accum), FMLA_ERR_ALIGNMENT, "dense_decode: o_accum must be 16-byte aligned");
  FMLA_REQUIRE((reinterpret_cast<uintptr_t>(a->sched_meta) & 31u) == 0, FMLA_ERR_ALIGNMENT, "dense_decode: scheduler metadata must be 32-byte aligned");
  FMLA_REQUIRE(tc_supported(a->h_q), FMLA_ERR_UNSUPPORTED, "dense_decode: the tensor-core kernel needs h_q to be a multiple of 64 (got %d)", a->h_q);
  FMLA_REQUIRE(a->sm_scale > 0.f, FMLA_ERR_UNSUPPORTED, "dense_decode: the softmax scale must be positive (got %g)", (double)a->sm_scale);
  DeviceInfo info;
  if (int rc = device_info(a->device, &info)) return rc;
  DeviceGuard guard(a->device);
  FMLA_REQUIRE(guard.ok, FMLA_ERR_CUDA, "dense_decode: cannot switch to device %d", a->device);
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (int rc = launch_tc_dense_decode(*a, stream)) return rc;
  FmlaDecodeArgs c = {};          // what the combine kernel reads
  c.b = a->b; c.s_q = a->s_q; c.h_q = a->h_q;
  c.num_splits = a->num_splits; c.o_accum = a->o_accum; c.lse_accum = a->lse_accum;
  c.out = a->out; c.o_stride_b = a->o_stride_b; c.o_stride_s = a->o_stride_s; c.o_stride_h = a->o_stride_h;
  c.lse = a->lse; c.lse_stride_b = a->lse_stride_b; c.lse_stride_s = a->lse_stride_s;
  return launch_combine(c, stream);
}

int fmla_sparse_prefill_fwd(const FmlaPrefillArgs* a, void* cuda_stream) {
  FMLA_REQUIRE(a != nullptr, FMLA_ERR_INVALID_ARG, "sparse_prefill_fwd: null argument struct");
  FMLA_REQUIRE(a->s_q > 0 && a->s_kv > 0 && a->h_q > 0 && a->topk > 0, FMLA_ERR_INVALID_ARG,
               "sparse_prefill_fwd: s_q=%d s_kv=%d h_q=%d topk=%d must be positive", a->s_q, a->s_kv, a->h_q, a->topk);
  FMLA_REQUIRE(a->q && a->kv && a->indices && a->out && a->max_logits && a->lse, FMLA_ERR_INVALID_ARG,
               "sparse_prefill_fwd: q, kv, indices, out, max_logits and lse must be non-null");
  FMLA_REQUIRE(a->d_qk == 0 || a->d_qk == FMLA_D_QK || a->d_qk == FMLA_MODEL1_D_QK, FMLA_ERR_UNSUPPORTED,
               "sparse_prefill_fwd: d_qk must be 576 or 512 (got %d)", a->d_qk);
  FMLA_REQUIRE(aligned16(a->q) && a->q_stride_s % 8 == 0 && a->q_stride_h % 8 == 0, FMLA_ERR_ALIGNMENT,
               "sparse_prefill_fwd: q base and strides must be multiples of 16 bytes");
  FMLA_REQUIRE(aligned16(a->kv) && a->kv_stride_s % 8 == 0, FMLA_ERR_ALIGNMENT,
               "sparse_prefill_fwd: kv base and row stride must be multiples of 16 bytes");
  FMLA_REQUIRE(aligned16(a->out), FMLA_ERR_ALIGNMENT, "sparse_prefill_fwd: out must be 16-byte aligned");
  const int k = pick_kernel(a->kernel, a->h_q, "sparse_prefill_fwd");
  if (k < 0) return FMLA_ERR_UNSUPPORTED;
  DeviceInfo info;
  if (int rc = device_info(a->device, &info)) return rc;
  DeviceGuard guard(a->device);
  FMLA_REQUIRE(guard.ok, FMLA_ERR_CUDA, "sparse_prefill_fwd: cannot switch to device %d", a->device);
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  const bool use_tc = k == FMLA_KERNEL_TC && (a->kernel == FMLA_KERNEL_TC || a->sm_scale > 0.f);   // AUTO: see fmla_sparse_decode
  return use_tc ? launch_tc_prefill_fwd(*a, stream) : launch_simt_prefill_fwd(*a, stream);
}

int fmla_sparse_prefill_bwd(const FmlaPrefillBwdArgs* a, void* cuda_stream) {
  FMLA_REQUIRE(a != nullptr, FMLA_ERR_INVALID_ARG, "sparse_prefill_bwd: null argument struct");
  FMLA_REQUIRE(a->s_q > 0 && a->s_kv > 0 && a->h_q > 0 && a->topk > 0, FMLA_ERR_INVALID_ARG,
               "sparse_prefill_bwd: s_q=%d s_kv=%d h_q=%d topk=%d must be positive", a->s_q, a->s_kv, a->h_q, a->topk);
  FMLA_REQUIRE(a->q && a->kv && a->out && a->dout && a->lse && a->indices && a->dq && a->dkv_accum, FMLA_ERR_INVALID_ARG,
               "sparse_prefill_bwd: q, kv, out, dout, lse, indices, dq and dkv_accum must be non-null");
  FMLA_REQUIRE(aligned16(a->q) && a->q_stride_s % 8 == 0 && a->q_stride_h % 8 == 0 && aligned16(a->kv) &&
                   a->kv_stride_s % 8 == 0 && aligned16(a->dout) && a->do_stride_s % 8 == 0 && a->do_stride_h % 8 == 0 &&
                   aligned16(a->out) && aligned16(a->dq) && aligned16(a->dkv_accum) && aligned16(a->dkv),
               FMLA_ERR_ALIGNMENT, "sparse_prefill_bwd: tensor bases and strides must be multiples of 16 bytes");
  DeviceInfo info;
  if (int rc = device_info(a->device, &info)) return rc;
  DeviceGuard guard(a->device);
  FMLA_REQUIRE(guard.ok, FMLA_ERR_CUDA, "sparse_prefill_bwd: cannot switch to device %d", a->device);
  // AUTO: tensor cores when the head count allows it and the caller lent a workspace; TC: required.
  const bool tc_ok = tc_bwd_supported(a->h_q);
  if (a->kernel == FMLA_KERNEL_TC)
    FMLA_REQUIRE(tc_ok, FMLA_ERR_UNSUPPORTED, "sparse_prefill_bwd: the tensor-core kernels need h_q to be a multiple of 64 (got %d)", a->h_q);
  const bool use_tc = a->kernel == FMLA_KERNEL_TC || (a->kernel != FMLA_KERNEL_SIMT && tc_ok && a->workspace != nullptr);
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  return use_tc ? launch_tc_prefill_bwd(*a, stream) : launch_simt_prefill_bwd(*a, stream);
}

int fmla_set_option(int option, int value) {
  if (option == FMLA_OPTION_PLAIN_Q_LOADS) { tc_set_plain_q_loads(value); return FMLA_OK; }
  if (option == FMLA_OPTION_PLAIN_STORES) { tc_set_plain_stores(value); return FMLA_OK; }
  set_error("set_option: unknown option %d", option);
  return FMLA_ERR_INVALID_ARG;
}

int fmla_tensor_map_cache_stats(uint64_t* hits, uint64_t* misses) {
  FMLA_REQUIRE(hits && misses, FMLA_ERR_INVALID_ARG, "tensor_map_cache_stats: null output pointer");
  unsigned long long h = 0, m = 0;
  tc_map_cache_stats(&h, &m);
  *hits = h; *misses = m;
  return FMLA_OK;
}

int64_t fmla_sparse_prefill_bwd_workspace(int s_q, int h_q, int topk, int kernel) {
  if (kernel == FMLA_KERNEL_SIMT || !tc_bwd_supported(h_q) || s_q <= 0 || topk <= 0) return 0;
  return (int64_t)s_q * tc_bwd_groups(h_q) * tc_bwd_unit_bytes(topk);
}

}  // extern "C"
