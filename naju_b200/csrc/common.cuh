// Shared device helpers for the sm_100a gated-scan kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "naju_b200.h"

namespace naju {

constexpr int kDT = 128;        // channels per tile == threads per CTA of the SIMT kernels
constexpr int kThreads = 128;
constexpr int kWarps = kThreads / 32;

// Spin budget of every device-side wait: iterations of (poll + nanosleep).  About 0.2 s in
// the worst case, after which the waiter records NAJU_ST_LOOKBACK_TIMEOUT and carries on
// with whatever it has, so a kernel can never hang the device.
constexpr int kSpinLimit = 1 << 20;

// ---------------------------------------------------------------- dtype conversion
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

__host__ __device__ __forceinline__ int dtype_size(int dt) { return dt == NAJU_F32 ? 4 : 2; }

// runtime-typed scalar access (used only for the small B/C tiles and the finalize kernels)
__device__ __forceinline__ float load_dyn(const void* p, int dt, int64_t idx) {
  if (dt == NAJU_F32) return reinterpret_cast<const float*>(p)[idx];
  if (dt == NAJU_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[idx]);
  return __half2float(reinterpret_cast<const __half*>(p)[idx]);
}
__device__ __forceinline__ void store_dyn(void* p, int dt, int64_t idx, float v) {
  if (dt == NAJU_F32) reinterpret_cast<float*>(p)[idx] = v;
  else if (dt == NAJU_BF16) reinterpret_cast<__nv_bfloat16*>(p)[idx] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(p)[idx] = __float2half_rn(v);
}

// ---------------------------------------------------------------- gates
// sigmoid(x) and 1 - sigmoid(x) without cancellation: a = e^-x, f = 1/(1+a), 1-f = a f.
// ex2.approx + a fast reciprocal keep the relative error near 2 ulp, which matters because
// retention gates multiply up over hundreds of steps.
struct Gate { float s; float one_minus; };
__device__ __forceinline__ Gate gate(float x) {
  x = fmaxf(x, -80.f);  // e^80 is finite in fp32; sigmoid(-80) ~ 1.8e-35 either way
  const float a = __expf(-x);
  const float s = __fdividef(1.f, 1.f + a);
  return Gate{s, a * s};
}
__device__ __forceinline__ float sigmoid_f(float x) { return gate(x).s; }

// ---------------------------------------------------------------- memory ordering
__device__ __forceinline__ int ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Waits (bounded) until *flag != 0 and returns it; returns 0 if the budget ran out.
__device__ __forceinline__ int wait_flag(const int* flag) {
  int v = ld_acquire(flag);
  int spins = 0;
  while (v == 0 && spins < kSpinLimit) {
    __nanosleep(64);
    v = ld_acquire(flag);
    ++spins;
  }
  return v;
}

// ---------------------------------------------------------------- async tile movement
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  const unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// Copies a [rows][cols_valid] window of a row-major global tensor into a dense [rows][kDT]
// shared tile (zero fill beyond cols_valid).  16-byte cp.async where source and row stride
// allow it, element loads otherwise.
template <typename T>
__device__ __forceinline__ void load_tile_async(T* __restrict__ dst, const T* __restrict__ src,
                                                int64_t row_stride, int rows, int cols_valid,
                                                int tid) {
  constexpr int EPV = 16 / sizeof(T);
  constexpr int VPR = kDT / EPV;
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(src) & 15) == 0) && (row_stride % EPV == 0);
  for (int v = tid; v < rows * VPR; v += kThreads) {
    const int r = v / VPR, c = (v % VPR) * EPV;
    T* d = dst + r * kDT + c;
    const T* s = src + static_cast<int64_t>(r) * row_stride + c;
    if (vec_ok && c + EPV <= cols_valid) {
      cp_async16(d, s);
    } else {
#pragma unroll
      for (int e = 0; e < EPV; ++e) d[e] = (c + e < cols_valid) ? s[e] : from_f32<T>(0.f);
    }
  }
}

// The same tile from a TIME-contiguous source: element (row r, channel c) sits at
// src[c * chan_stride + r].  Thread c walks its channel's steps; plain stores, visible after the
// block barrier that follows the staging.  (The slow, general path for this layout: the walk-along-
// time tensor-core kernels take it natively.)
template <typename T>
__device__ __forceinline__ void load_tile_tmajor(T* __restrict__ dst, const T* __restrict__ src,
                                                 int64_t chan_stride, int rows, int cols_valid, int tid) {
  if (tid < kDT) {
    const T* s = src + static_cast<int64_t>(tid) * chan_stride;
    for (int r = 0; r < rows; ++r) dst[r * kDT + tid] = tid < cols_valid ? s[r] : from_f32<T>(0.f);
  }
}

// ... and the store to a TIME-contiguous destination: element (row r, channel c) goes to
// dst[c * chan_stride + r].
template <typename T>
__device__ __forceinline__ void store_tile_tmajor(T* __restrict__ dst, const T* __restrict__ src,
                                                  int64_t chan_stride, int rows, int cols_valid, int tid) {
  if (tid < cols_valid) {
    T* d = dst + static_cast<int64_t>(tid) * chan_stride;
    for (int r = 0; r < rows; ++r) d[r] = src[r * kDT + tid];
  }
}

// Writes a dense [rows][kDT] shared tile to a row-major global tensor window.
template <typename T>
__device__ __forceinline__ void store_tile(T* __restrict__ dst, const T* __restrict__ src,
                                           int64_t row_stride, int rows, int cols_valid, int tid) {
  constexpr int EPV = 16 / sizeof(T);
  constexpr int VPR = kDT / EPV;
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) && (row_stride % EPV == 0);
  for (int v = tid; v < rows * VPR; v += kThreads) {
    const int r = v / VPR, c = (v % VPR) * EPV;
    const T* s = src + r * kDT + c;
    T* d = dst + static_cast<int64_t>(r) * row_stride + c;
    if (vec_ok && c + EPV <= cols_valid) {
      *reinterpret_cast<uint4*>(d) = *reinterpret_cast<const uint4*>(s);
    } else {
#pragma unroll
      for (int e = 0; e < EPV; ++e)
        if (c + e < cols_valid) d[e] = s[e];
    }
  }
}

// Loads `rows` rows of a [*, N] tensor of runtime dtype into a dense fp32 [rows][NS] shared
// tile, zero padded for n >= N.
template <int NS>
__device__ __forceinline__ void load_bc_tile(float* __restrict__ dst, const void* __restrict__ src,
                                             int dt, int64_t base, int64_t row_stride, int rows,
                                             int N, int tid) {
  for (int e = tid; e < rows * NS; e += kThreads) {
    const int r = e / NS, n = e % NS;
    dst[e] = (n < N) ? load_dyn(src, dt, base + static_cast<int64_t>(r) * row_stride + n) : 0.f;
  }
}

// ---------------------------------------------------------------- warp reduce-scatter
// Sums v[0..NS) over the 32 lanes of a warp.  On return lane L holds, in v[0..out_count),
// the totals of the entries n = out_base(L) + j.  NS=16: one value, n = L>>1 (lanes 2k and
// 2k+1 hold the same total).  NS>=32: NS/32 values.  Fixed order, hence deterministic.
template <int NS>
struct WarpRS {
  static constexpr int out_count = (NS >= 32) ? NS / 32 : 1;
  __device__ static __forceinline__ int out_base(int lane) {
    int base = 0, cnt = NS;
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) {
      if (cnt > 1) {
        cnt >>= 1;
        if (lane & m) base += cnt;
      }
    }
    return base;
  }
  __device__ static __forceinline__ void run(float (&v)[NS], int lane) {
    int cnt = NS;
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) {
      if (cnt > 1) {
        const int half = cnt >> 1;
        const bool upper = (lane & m) != 0;
#pragma unroll
        for (int j = 0; j < NS / 2; ++j) {
          if (j < half) {
            const float send = upper ? v[j] : v[j + half];
            const float keep = upper ? v[j + half] : v[j];
            v[j] = keep + __shfl_xor_sync(0xffffffffu, send, m);
          }
        }
        cnt = half;
      } else {
        v[0] += __shfl_xor_sync(0xffffffffu, v[0], m);
      }
    }
  }
};

}  // namespace naju
