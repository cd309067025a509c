// Shared host/device helpers for the flashmla_b200 kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/flashmla_b200.h"

namespace fmla {

// ---- error reporting -------------------------------------------------------------------------
void set_error(const char* fmt, ...);   // stores a thread-local message (api.cu)

#define FMLA_REQUIRE(cond, code, ...)            \
  do {                                           \
    if (!(cond)) {                               \
      ::fmla::set_error(__VA_ARGS__);            \
      return (code);                             \
    }                                            \
  } while (0)

#define FMLA_CUDA(call)                                                                          \
  do {                                                                                           \
    cudaError_t err__ = (call);                                                                  \
    if (err__ != cudaSuccess) {                                                                  \
      ::fmla::set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(err__), __FILE__, __LINE__); \
      return FMLA_ERR_CUDA;                                                                      \
    }                                                                                            \
  } while (0)

// RAII device switch: entry points run on args->device and restore the caller's device.
struct DeviceGuard {
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
    if (prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
  }
  ~DeviceGuard() {
    int cur = -1;
    if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
  }
};

// ---- constants -------------------------------------------------------------------------------
constexpr int D_QK = FMLA_D_QK;
constexpr int D_V = FMLA_D_V;
constexpr int D_NOPE = 512;
constexpr int D_ROPE = 64;
constexpr int ROW_BYTES = FMLA_ROW_BYTES;
constexpr int SCALE_OFF = 512;
constexpr int ROPE_OFF = 528;
// MODEL1 cache blocks: [page x 576 data bytes (448 e4m3 | 64 bf16)] [page x 8 scale bytes (7 e8m0 | pad)]
constexpr int M1_D_QK = FMLA_MODEL1_D_QK, M1_D_NOPE = 448, M1_DATA_BYTES = FMLA_MODEL1_DATA_BYTES, M1_ROW_BYTES = FMLA_MODEL1_ROW_BYTES;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

// One partition record written by the tile scheduler and read by the decode kernels.
struct __align__(32) SchedRecord {
  int begin_req, end_req;      // both inclusive
  int begin_block, end_block;  // inclusive, exclusive (of begin_req / end_req respectively)
  int begin_split;             // split index of begin_req handled by this partition
  int first_split, last_split; // whether begin_req / end_req is shared with other partitions
  int pad;
};
static_assert(sizeof(SchedRecord) == 4 * FMLA_SCHED_META_INTS, "record is 8 int32");

// ---- launchers implemented in the other translation units -------------------------------------
int launch_sched_meta(const FmlaSchedArgs& a, cudaStream_t stream);
int launch_combine(const FmlaDecodeArgs& a, cudaStream_t stream);
int launch_simt_decode(const FmlaDecodeArgs& a, cudaStream_t stream);
int launch_simt_prefill_fwd(const FmlaPrefillArgs& a, cudaStream_t stream);
int launch_simt_prefill_bwd(const FmlaPrefillBwdArgs& a, cudaStream_t stream);
// tensor-core (tcgen05) kernels
bool tc_supported(int h_q);
void tc_set_plain_q_loads(int on);      // diagnostic: Q through plain loads instead of TMA tiles
void tc_set_plain_stores(int on);       // diagnostic: results through plain stores instead of TMA box stores
void tc_map_cache_stats(unsigned long long* hits, unsigned long long* misses);
int tc_decode_plan(int num_sms, int h_q, int s_q, int* num_sm_parts, int* fixed_overhead_blocks, int* block_topk);
bool tc_decode_supported(const FmlaDecodeArgs& a);      // stride and scale preconditions of the tensor-core decode kernel
int launch_tc_decode(const FmlaDecodeArgs& a, cudaStream_t stream);
int launch_tc_dense_decode(const FmlaDenseDecodeArgs& a, cudaStream_t stream);
int launch_tc_prefill_fwd(const FmlaPrefillArgs& a, cudaStream_t stream);
bool tc_bwd_supported(int h_q);
int tc_bwd_groups(int h_q);             // units (groups of up to 128 heads) per query token
int64_t tc_bwd_unit_bytes(int topk);   // workspace per (query token, group of 128 heads)
int launch_tc_prefill_bwd(const FmlaPrefillBwdArgs& a, cudaStream_t stream);

// ---- small device helpers --------------------------------------------------------------------
#ifdef __CUDACC__
__device__ __forceinline__ float bf16_bits_to_float(uint32_t hi16) { return __uint_as_float(hi16 << 16); }

// Two packed e4m3 bytes -> two floats (exact).
__device__ __forceinline__ float2 e4m3x2_to_float2(uint16_t v) {
  __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)v, __NV_E4M3);
  return __half22float2(*reinterpret_cast<__half2*>(&h));
}

// e8m0 scale byte -> float 2^(byte-127); 0 encodes 2^-127 (a subnormal float), 255 encodes NaN.
__device__ __forceinline__ float e8m0_to_float(uint32_t byte) {
  uint32_t bits = byte == 0 ? 0x00400000u : (byte == 255u ? 0x7fc00000u : (byte << 23));
  return __uint_as_float(bits);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ uint4 ldg_nc_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ldg_nc_8(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
#endif

}  // namespace fmla
