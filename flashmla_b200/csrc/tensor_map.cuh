// Host-side helpers shared by the tensor-core launchers: tensor-map encoding through the runtime's driver entry
// point table (no direct libcuda dependency) with a small cache, and once-per-device kernel attribute set-up.
//
// Encoding a tensor map costs a driver call of a few microseconds; a serving loop calls the same entry point with the
// same buffers (KV pool, cached q / output buffers of a CUDA graph) over and over, so encoded maps are kept in a table
// keyed by everything that goes into the encoding.  A hit copies 128 bytes.  The table is process-wide, guarded by a
// mutex, and replaces its oldest entry when full; the descriptors hold addresses only, so an entry that outlives its
// buffer is harmless until the same key is asked for again, when it is exactly the right descriptor for the new buffer.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstring>
#include <mutex>

namespace fmla {
namespace tmap {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static std::once_flag once;
  static EncodeTiledFn fn = nullptr;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) == cudaSuccess &&
        res == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

struct Key {
  const void* base;
  uint32_t dtype, rank, swizzle, pad;
  uint64_t dims[4], strides[3];
  uint32_t box[4];
};

struct Cache {
  static constexpr int N = 64;
  std::mutex mu;
  Key keys[N];
  CUtensorMap maps[N];
  int used = 0, next = 0;
  unsigned long long hits = 0, misses = 0;
};
inline Cache& cache() {
  static Cache c;
  return c;
}

// Encodes (or looks up) a tiled map: `rank` dims innermost first, byte strides for dims 1.., element strides 1,
// zero fill outside the tensor.  Returns the driver's result code (CUDA_SUCCESS = 0), or -1 without an encoder.
inline int encode(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int rank, const uint64_t* dims,
                  const uint64_t* strides, const uint32_t* box, CUtensorMapSwizzle swizzle) {
  Key k;
  std::memset(&k, 0, sizeof(k));
  k.base = base; k.dtype = (uint32_t)dtype; k.rank = (uint32_t)rank; k.swizzle = (uint32_t)swizzle;
  for (int i = 0; i < rank; ++i) { k.dims[i] = dims[i]; k.box[i] = box[i]; }
  for (int i = 0; i + 1 < rank; ++i) k.strides[i] = strides[i];
  Cache& c = cache();
  {
    std::lock_guard<std::mutex> lock(c.mu);
    for (int i = 0; i < c.used; ++i)
      if (std::memcmp(&c.keys[i], &k, sizeof(k)) == 0) { *out = c.maps[i]; ++c.hits; return 0; }
  }
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t d[4], s[3];
  cuuint32_t b[4], e[4] = {1, 1, 1, 1};
  for (int i = 0; i < rank; ++i) { d[i] = dims[i]; b[i] = box[i]; }
  for (int i = 0; i + 1 < rank; ++i) s[i] = strides[i];
  const CUresult rc = fn(out, dtype, (cuuint32_t)rank, const_cast<void*>(base), d, s, b, e, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return (int)rc;
  std::lock_guard<std::mutex> lock(c.mu);
  const int slot = c.used < Cache::N ? c.used++ : (c.next++ % Cache::N);
  c.keys[slot] = k;
  c.maps[slot] = *out;
  ++c.misses;
  return 0;
}

// Runs `set` (which sets a kernel's function attributes for the current device) once per device ordinal.
struct PerDeviceOnce {
  std::mutex mu;
  bool done[64] = {};
  template <class F>
  cudaError_t run(F set) {
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= 64) return set();
    std::lock_guard<std::mutex> lock(mu);
    if (done[dev]) return cudaSuccess;
    err = set();
    if (err == cudaSuccess) done[dev] = true;
    return err;
  }
};

}  // namespace tmap
}  // namespace fmla
