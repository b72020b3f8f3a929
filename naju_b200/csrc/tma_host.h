// Host-side helpers shared by the TMA-fed kernels' launchers: the tensor-map encoder (looked up
// once through the runtime, no link against libcuda) and the SM count of the current device.
// Both initialisations are thread-safe (autograd runs backward on a worker thread).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "naju_b200.h"

namespace naju {
namespace tmah {

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                             const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeFn lookup_encode_fn() {
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
      qres == cudaDriverEntryPointSuccess)
    return reinterpret_cast<EncodeFn>(sym);
  return nullptr;
}

// (a function-local static is initialised exactly once, even when two threads race to it)
inline EncodeFn encode_fn() {
  static const EncodeFn fn = lookup_encode_fn();
  return fn;
}

inline CUtensorMapDataType tm_dtype(int dt) {
  return dt == NAJU_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                        : dt == NAJU_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
}

// Map of a [B][T][inner] tensor with element strides (sb, st, 1); box = (box_inner, box_t, 1).
// False when TMA cannot describe it (base or strides not multiples of 16 bytes, overlapping rows).
inline bool make_map(CUtensorMap* m, const void* base, int dt, int64_t B, int64_t T, int64_t inner, int64_t sb,
                     int64_t st, int box_inner, int box_t) {
  const int es = dt == NAJU_F32 ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return false;
  if ((st * es) % 16 != 0 || (sb * es) % 16 != 0 || (box_inner * es) % 16 != 0) return false;
  if (B > 1 && sb < st) return false;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(T), static_cast<cuuint64_t>(B)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(st * es), static_cast<cuuint64_t>((B > 1 ? sb : st * T) * es)};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_t), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const EncodeFn fn = encode_fn();
  if (!fn) return false;
  return fn(m, tm_dtype(dt), 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Map of a [B][T][D] tensor stored TIME-contiguous, element strides (sb, 1, sd): TMA dimensions
// (T, D, B), box = (box_t, box_d, 1); a tile lands in shared memory as [box_d][box_t].
inline bool make_map_tmajor(CUtensorMap* m, const void* base, int dt, int64_t B, int64_t T, int64_t D, int64_t sb,
                            int64_t sd, int box_t, int box_d) {
  const int es = dt == NAJU_F32 ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return false;
  if ((sd * es) % 16 != 0 || (sb * es) % 16 != 0 || (box_t * es) % 16 != 0) return false;
  if (sd < T || (B > 1 && sb < sd)) return false;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(T), static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(B)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(sd * es), static_cast<cuuint64_t>((B > 1 ? sb : sd * D) * es)};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(box_t), static_cast<cuuint32_t>(box_d), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const EncodeFn fn = encode_fn();
  if (!fn) return false;
  return fn(m, tm_dtype(dt), 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// SM count of the CURRENT device (cached per device ordinal; a racing first call at worst asks twice).
inline int sm_count() {
  constexpr int kMaxDev = 64;
  static int cache[kMaxDev] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev >= 0 && dev < kMaxDev) {
    const int c = __atomic_load_n(&cache[dev], __ATOMIC_RELAXED);
    if (c > 0) return c;
  }
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  if (dev >= 0 && dev < kMaxDev) __atomic_store_n(&cache[dev], n, __ATOMIC_RELAXED);
  return n;
}

}  // namespace tmah
}  // namespace naju
