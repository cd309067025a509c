// The step before the attention path: writing the paged KV cache.
//   * kv_quantize_kernel turns bf16 rows [576] into the 656-byte cache rows the decode kernels read
//     (V32: 512 e4m3 | 4 fp32 scales per 128 | 64 bf16 RoPE; MXFP8: 512 e4m3 | 16 e8m0 scale bytes per 32 | 64 bf16),
//     byte for byte what the reference's test quantiser produces (tests/quant.py:17-18, 35-53): the scale of a
//     tile is the smallest power of two >= max(amax / 448, 1e-4), values are divided by it and rounded to
//     e4m3 to nearest even.
//   * cache_index_kernel maps logical token positions to in-cache row indices through the block table
//     (tests/quant.py:126-158): row = block_table[b, pos / page] * page + pos % page, -1 stays -1.
// Both are HBM-bound byte work: one warp per row (1152 bytes read, 656 written), 16-byte accesses.
#include <cuda_fp8.h>

#include "common.cuh"

namespace fmla {
namespace {

constexpr int QUANT_WARPS = 8;

// Smallest power of two >= max(amax / 448, 1e-4) as its fp32 bit pattern.  The division is IEEE (the
// library is built with fast-math, which would replace the operator by an approximation).
__device__ __forceinline__ uint32_t pow2_scale_bits(float amax) {
  const float v = fmaxf(__fdiv_rn(amax, 448.f), 1e-4f);
  const uint32_t bits = __float_as_uint(v);
  return (bits & 0x7f800000u) + ((bits & 0x007fffffu) ? 0x00800000u : 0u);
}

__global__ void __launch_bounds__(32 * QUANT_WARPS)
kv_quantize_kernel(const __nv_bfloat16* __restrict__ src, int64_t src_stride, uint8_t* __restrict__ dst, int64_t page,
                   int64_t dst_block_stride, int64_t n_rows, int layout) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * QUANT_WARPS + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const __nv_bfloat16* in = src + row * src_stride;
  uint8_t* out = dst + (row / page) * dst_block_stride + (row % page) * ROW_BYTES;

  // lane l holds the 16-byte chunks l and l + 32 of the NoPE part (8 values each)
  uint4 raw[2];
  float amax[2];
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    raw[k] = ldg_nc_16(in + 8 * (lane + 32 * k));
    const uint32_t w[4] = {raw[k].x, raw[k].y, raw[k].z, raw[k].w};
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) m = fmaxf(m, fmaxf(fabsf(bf16_bits_to_float(w[i] & 0xffffu)), fabsf(bf16_bits_to_float(w[i] >> 16))));
    amax[k] = m;
  }
  // tile maximum: V32 tiles are 128 values = 16 consecutive lanes, MXFP8 tiles 32 values = 4 consecutive lanes
  const int span = layout == FMLA_LAYOUT_V32 ? 16 : 4;
#pragma unroll
  for (int k = 0; k < 2; ++k)
    for (int d = 1; d < span; d <<= 1) amax[k] = fmaxf(amax[k], __shfl_xor_sync(0xffffffffu, amax[k], d));

#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const uint32_t sbits = pow2_scale_bits(amax[k]);
    const float inv = __uint_as_float(0x7f000000u - sbits);          // 1 / 2^e = 2^-e, exact
    const uint32_t w[4] = {raw[k].x, raw[k].y, raw[k].z, raw[k].w};
    uint32_t q[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t lo = __nv_cvt_float_to_fp8(bf16_bits_to_float(w[i] & 0xffffu) * inv, __NV_SATFINITE, __NV_E4M3);
      const uint32_t hi = __nv_cvt_float_to_fp8(bf16_bits_to_float(w[i] >> 16) * inv, __NV_SATFINITE, __NV_E4M3);
      q[i >> 1] |= (lo | (hi << 8)) << (16 * (i & 1));
    }
    *reinterpret_cast<uint2*>(out + 8 * (lane + 32 * k)) = make_uint2(q[0], q[1]);
    const int chunk = lane + 32 * k;                                   // values [8 chunk, 8 chunk + 8)
    if (layout == FMLA_LAYOUT_V32) {
      if ((chunk & 15) == 0) *reinterpret_cast<uint32_t*>(out + 512 + 4 * (chunk >> 4)) = sbits;
    } else {
      if ((chunk & 3) == 0) out[512 + (chunk >> 2)] = (uint8_t)(sbits >> 23);   // e8m0 = the biased exponent
    }
  }
  if (lane < 8) *reinterpret_cast<uint4*>(out + 528 + 16 * lane) = ldg_nc_16(in + 512 + 8 * lane);
}

// MODEL1 (tests/quant.py:55-75): bf16 rows [512] -> per cache block [page x (448 e4m3 | 64 bf16)] [page x (7 e8m0 | pad)].
// One warp per row; lane l holds the 16-byte chunks l and l + 32 of the 64 (chunks 0..55 NoPE, 56..63 RoPE); a scale
// covers 64 values = 8 consecutive lanes.
__global__ void __launch_bounds__(32 * QUANT_WARPS)
kv_quantize_model1_kernel(const __nv_bfloat16* __restrict__ src, int64_t src_stride, uint8_t* __restrict__ dst, int64_t page,
                          int64_t dst_block_stride, int64_t n_rows) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * QUANT_WARPS + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const __nv_bfloat16* in = src + row * src_stride;
  uint8_t* block = dst + (row / page) * dst_block_stride;
  uint8_t* out = block + (row % page) * M1_DATA_BYTES;
  uint8_t* scales = block + page * M1_DATA_BYTES + (row % page) * 8;
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int chunk = lane + 32 * k;
    const uint4 raw = ldg_nc_16(in + 8 * chunk);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) amax = fmaxf(amax, fmaxf(fabsf(bf16_bits_to_float(w[i] & 0xffffu)), fabsf(bf16_bits_to_float(w[i] >> 16))));
    for (int d = 1; d < 8; d <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
    if (chunk >= 56) {                                                   // RoPE: copied verbatim behind the 448 bytes
      *reinterpret_cast<uint4*>(out + M1_D_NOPE + 16 * (chunk - 56)) = raw;
      continue;
    }
    const uint32_t sbits = pow2_scale_bits(amax);
    const float inv = __uint_as_float(0x7f000000u - sbits);              // 1 / 2^e = 2^-e, exact
    uint32_t q[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t lo = __nv_cvt_float_to_fp8(bf16_bits_to_float(w[i] & 0xffffu) * inv, __NV_SATFINITE, __NV_E4M3);
      const uint32_t hi = __nv_cvt_float_to_fp8(bf16_bits_to_float(w[i] >> 16) * inv, __NV_SATFINITE, __NV_E4M3);
      q[i >> 1] |= (lo | (hi << 8)) << (16 * (i & 1));
    }
    *reinterpret_cast<uint2*>(out + 8 * chunk) = make_uint2(q[0], q[1]);
    if ((chunk & 7) == 0) scales[chunk >> 3] = (uint8_t)(sbits >> 23);   // e8m0 = the biased exponent
  }
  if (lane == 0) scales[7] = 0;
}

__global__ void cache_index_kernel(const int* __restrict__ pos, const int* __restrict__ block_table, int* __restrict__ out,
                                   int64_t per_request, int64_t total, int page, int max_pages) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int p = pos[i];
  int r = -1;
  if (p >= 0) {
    const int64_t b = i / per_request;
    const int pg = p / page;
    if (pg < max_pages) r = block_table[b * max_pages + pg] * page + (p - pg * page);
  }
  out[i] = r;
}

}  // namespace
}  // namespace fmla

using namespace fmla;

extern "C" int fmla_kv_quantize(const FmlaKvQuantArgs* a, void* cuda_stream) {
  FMLA_REQUIRE(a != nullptr, FMLA_ERR_INVALID_ARG, "kv_quantize: null argument struct");
  FMLA_REQUIRE(a->n_rows > 0 && a->page_block_size > 0, FMLA_ERR_INVALID_ARG,
               "kv_quantize: n_rows=%lld page_block_size=%lld must be positive", (long long)a->n_rows, (long long)a->page_block_size);
  FMLA_REQUIRE(a->layout == FMLA_LAYOUT_V32 || a->layout == FMLA_LAYOUT_MXFP8 || a->layout == FMLA_LAYOUT_MODEL1, FMLA_ERR_UNSUPPORTED,
               "kv_quantize: unknown KV layout %d", a->layout);
  const bool m1 = a->layout == FMLA_LAYOUT_MODEL1;
  const int d_qk = m1 ? M1_D_QK : D_QK;
  const int64_t row_bytes = m1 ? M1_ROW_BYTES : ROW_BYTES;
  FMLA_REQUIRE(a->kv && a->rows, FMLA_ERR_INVALID_ARG, "kv_quantize: kv and rows must be non-null");
  FMLA_REQUIRE((reinterpret_cast<uintptr_t>(a->kv) & 15u) == 0 && a->kv_stride_row % 8 == 0 && a->kv_stride_row >= d_qk, FMLA_ERR_ALIGNMENT,
               "kv_quantize: kv must be 16-byte aligned with a row stride that is a multiple of 8 elements and at least %d", d_qk);
  FMLA_REQUIRE((reinterpret_cast<uintptr_t>(a->rows) & 15u) == 0 && a->rows_stride_block % 16 == 0 &&
                   a->rows_stride_block >= a->page_block_size * row_bytes, FMLA_ERR_ALIGNMENT,
               "kv_quantize: rows must be 16-byte aligned with a block stride that is a multiple of 16 bytes and at least page_block_size*%lld",
               (long long)row_bytes);
  DeviceGuard guard(a->device);
  FMLA_REQUIRE(guard.ok, FMLA_ERR_CUDA, "kv_quantize: cannot switch to device %d", a->device);
  const int64_t blocks = (a->n_rows + QUANT_WARPS - 1) / QUANT_WARPS;
  FMLA_REQUIRE(blocks <= 0x7fffffffLL, FMLA_ERR_UNSUPPORTED, "kv_quantize: too many rows for one launch");
  if (m1)
    kv_quantize_model1_kernel<<<(unsigned)blocks, 32 * QUANT_WARPS, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
        static_cast<const __nv_bfloat16*>(a->kv), a->kv_stride_row, static_cast<uint8_t*>(a->rows), a->page_block_size,
        a->rows_stride_block, a->n_rows);
  else
    kv_quantize_kernel<<<(unsigned)blocks, 32 * QUANT_WARPS, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
        static_cast<const __nv_bfloat16*>(a->kv), a->kv_stride_row, static_cast<uint8_t*>(a->rows), a->page_block_size,
        a->rows_stride_block, a->n_rows, a->layout);
  FMLA_CUDA(cudaGetLastError());
  return FMLA_OK;
}

extern "C" int fmla_cache_indices(const FmlaCacheIndexArgs* a, void* cuda_stream) {
  FMLA_REQUIRE(a != nullptr, FMLA_ERR_INVALID_ARG, "cache_indices: null argument struct");
  FMLA_REQUIRE(a->b > 0 && a->per_request > 0 && a->page_block_size > 0 && a->max_pages > 0, FMLA_ERR_INVALID_ARG,
               "cache_indices: b=%d per_request=%lld page_block_size=%d max_pages=%d must be positive", a->b,
               (long long)a->per_request, a->page_block_size, a->max_pages);
  FMLA_REQUIRE(a->positions && a->block_table && a->indices, FMLA_ERR_INVALID_ARG, "cache_indices: null pointer");
  DeviceGuard guard(a->device);
  FMLA_REQUIRE(guard.ok, FMLA_ERR_CUDA, "cache_indices: cannot switch to device %d", a->device);
  const int64_t total = (int64_t)a->b * a->per_request;
  const int64_t blocks = (total + 255) / 256;
  FMLA_REQUIRE(blocks <= 0x7fffffffLL, FMLA_ERR_UNSUPPORTED, "cache_indices: too many indices for one launch");
  cache_index_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      a->positions, a->block_table, a->indices, a->per_request, total, a->page_block_size, a->max_pages);
  FMLA_CUDA(cudaGetLastError());
  return FMLA_OK;
}
