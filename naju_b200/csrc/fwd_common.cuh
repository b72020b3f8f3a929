// Tile-level building blocks of the forward scan shared by the exact recurrent kernel and
// by the tensor-core kernel's per-tile exact path.
#pragma once

#include "common.cuh"
#include "params.h"

namespace naju {

// Tile coordinates handed out by the time-major ticket.
struct TileCoord {
  int64_t tile;
  int c, rem, b, dt, per_chunk, t0, len, d0, cols, d;
  bool d_ok;
};

template <int TC>
__device__ __forceinline__ bool decode_tile(unsigned ticket, int B, int T, int D, int nchunks,
                                            int ndt, int tid, TileCoord& tc) {
  tc.tile = ticket;
  tc.per_chunk = B * ndt;
  tc.c = static_cast<int>(ticket / tc.per_chunk);
  tc.rem = static_cast<int>(ticket % tc.per_chunk);
  tc.b = tc.rem / ndt;
  tc.dt = tc.rem % ndt;
  tc.t0 = tc.c * TC;
  tc.len = min(TC, T - tc.t0);
  tc.d0 = tc.dt * kDT;
  tc.cols = min(kDT, D - tc.d0);
  tc.d = tc.d0 + tid;
  tc.d_ok = tc.d < D;
  return tc.c < nchunks;
}

// pass 1: local scan of the staged tile from a zero state -> x = chunk-end state, P = prod f
template <typename TA, typename TG, int NS>
__device__ __forceinline__ void tile_pass1(const TA* s_u, const TG* s_fl, const TG* s_il,
                                           const float* s_B, int len, int tid, float (&x)[NS],
                                           float& P) {
#pragma unroll
  for (int n = 0; n < NS; ++n) x[n] = 0.f;
  P = 1.f;
  for (int t = 0; t < len; ++t) {
    const float f = sigmoid_f(to_f32(s_fl[t * kDT + tid]));
    const float w = sigmoid_f(to_f32(s_il[t * kDT + tid])) * to_f32(s_u[t * kDT + tid]);
    P *= f;
    const float4* Bt = reinterpret_cast<const float4*>(s_B + t * NS);
#pragma unroll
    for (int q = 0; q < NS / 4; ++q) {
      const float4 bv = Bt[q];
      x[4 * q + 0] = fmaf(f, x[4 * q + 0], w * bv.x);
      x[4 * q + 1] = fmaf(f, x[4 * q + 1], w * bv.y);
      x[4 * q + 2] = fmaf(f, x[4 * q + 2], w * bv.z);
      x[4 * q + 3] = fmaf(f, x[4 * q + 3], w * bv.w);
    }
  }
}

// Carry across chunks.  In: (P, S) the tile's local aggregate.  Out: h = state entering the
// chunk, Pin = product of f from t=0 to the chunk start.  Publishes the aggregate, resolves
// the carry-in by bounded decoupled look-back and publishes the inclusive chunk-end state
// (the backward's checkpoint).  Must be called by all threads of the CTA.
// NAMED = false: all threads of the CTA take part (__syncthreads).  NAMED = true: only the first
// 128 threads do (named barrier 1), for kernels whose other warps have other roles.
template <bool NAMED>
__device__ __forceinline__ void carry_sync() {
  if constexpr (NAMED) asm volatile("bar.sync 1, 128;" ::: "memory");
  else __syncthreads();
}

template <int NS, bool NAMED = false>
__device__ __forceinline__ void carry_lookback(const FwdParams& p, const TileCoord& tc, int tid,
                                               const float (&S)[NS], float P, float (&h)[NS],
                                               float& Pin) {
  const int64_t slot = tc.tile * kDT + tid;
  Pin = 1.f;
  if (tc.c == 0) {
#pragma unroll
    for (int n = 0; n < NS; ++n)
      h[n] = (p.h0 != nullptr && tc.d_ok && n < p.N)
                 ? p.h0[(static_cast<int64_t>(tc.b) * p.D + tc.d) * p.N + n] : 0.f;
  } else {
    p.aggP[slot] = P;
    float4* dstS = reinterpret_cast<float4*>(p.aggS + slot * NS);
#pragma unroll
    for (int q = 0; q < NS / 4; ++q)
      dstS[q] = make_float4(S[4 * q], S[4 * q + 1], S[4 * q + 2], S[4 * q + 3]);
    carry_sync<NAMED>();
    if (tid == 0) {
      __threadfence();  // cumulative: orders every thread's stores above (seen through the barrier)
      st_release(p.flags + tc.tile, 1);
    }

    float accP = 1.f;
#pragma unroll
    for (int n = 0; n < NS; ++n) h[n] = 0.f;
    for (int j = tc.c - 1; j >= 0; --j) {
      const int64_t jt = static_cast<int64_t>(j) * tc.per_chunk + tc.rem;
      const int64_t js = jt * kDT + tid;
      const int st = wait_flag(p.flags + jt);
      if (st == 0) {
        atomicOr(&p.hdr->status, NAJU_ST_LOOKBACK_TIMEOUT);
        break;
      }
      const float4* src = reinterpret_cast<const float4*>((st == 2 ? p.ckS : p.aggS) + js * NS);
#pragma unroll
      for (int q = 0; q < NS / 4; ++q) {
        const float4 v = __ldcg(src + q);
        h[4 * q + 0] = fmaf(accP, v.x, h[4 * q + 0]);
        h[4 * q + 1] = fmaf(accP, v.y, h[4 * q + 1]);
        h[4 * q + 2] = fmaf(accP, v.z, h[4 * q + 2]);
        h[4 * q + 3] = fmaf(accP, v.w, h[4 * q + 3]);
      }
      if (st == 2) {
        Pin = accP * __ldcg(p.ckP + js);
        break;
      }
      accP *= __ldcg(p.aggP + js);
    }
  }
  float4* dstS = reinterpret_cast<float4*>(p.ckS + slot * NS);
#pragma unroll
  for (int q = 0; q < NS / 4; ++q)
    dstS[q] = make_float4(fmaf(P, h[4 * q + 0], S[4 * q + 0]), fmaf(P, h[4 * q + 1], S[4 * q + 1]),
                          fmaf(P, h[4 * q + 2], S[4 * q + 2]), fmaf(P, h[4 * q + 3], S[4 * q + 3]));
  p.ckP[slot] = P * Pin;
  carry_sync<NAMED>();
  if (tid == 0) {
    __threadfence();
    st_release(p.flags + tc.tile, 2);
  }
}

// pass 2: scan from the true carry-in, y written into the u tile; x ends as the chunk-end state
template <typename TA, typename TG, int NS>
__device__ __forceinline__ void tile_pass2(TA* s_u, const TG* s_fl, const TG* s_il,
                                           const float* s_B, const float* s_C, int len, int tid,
                                           float Dv, float (&x)[NS]) {
  for (int t = 0; t < len; ++t) {
    const float ut = to_f32(s_u[t * kDT + tid]);
    const float f = sigmoid_f(to_f32(s_fl[t * kDT + tid]));
    const float w = sigmoid_f(to_f32(s_il[t * kDT + tid])) * ut;
    const float4* Bt = reinterpret_cast<const float4*>(s_B + t * NS);
    const float4* Ct = reinterpret_cast<const float4*>(s_C + t * NS);
    float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
    for (int q = 0; q < NS / 4; ++q) {
      const float4 bv = Bt[q];
      const float4 cv = Ct[q];
      x[4 * q + 0] = fmaf(f, x[4 * q + 0], w * bv.x);
      x[4 * q + 1] = fmaf(f, x[4 * q + 1], w * bv.y);
      x[4 * q + 2] = fmaf(f, x[4 * q + 2], w * bv.z);
      x[4 * q + 3] = fmaf(f, x[4 * q + 3], w * bv.w);
      acc0 = fmaf(cv.x, x[4 * q + 0], acc0);
      acc1 = fmaf(cv.y, x[4 * q + 1], acc1);
      acc0 = fmaf(cv.z, x[4 * q + 2], acc0);
      acc1 = fmaf(cv.w, x[4 * q + 3], acc1);
    }
    s_u[t * kDT + tid] = from_f32<TA>(fmaf(Dv, ut, acc0 + acc1));
  }
}

// final state / total decay outputs of the last chunk
template <int NS>
__device__ __forceinline__ void write_final(const FwdParams& p, const TileCoord& tc,
                                            const float (&xend)[NS], float Ptot) {
  if (tc.c == p.nchunks - 1 && tc.d_ok) {
    if (p.hT != nullptr) {
      float* o = p.hT + (static_cast<int64_t>(tc.b) * p.D + tc.d) * p.N;
#pragma unroll
      for (int n = 0; n < NS; ++n)
        if (n < p.N) o[n] = xend[n];
    }
    if (p.pT != nullptr) p.pT[static_cast<int64_t>(tc.b) * p.D + tc.d] = Ptot;
  }
}

}  // namespace naju
