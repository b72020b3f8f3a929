// Forward gated scan, exact recurrent form (any gate logit).
//
//   x_t[n] = f_t x_{t-1}[n] + (i_t u_t) B_t[n],   y_t = sum_n C_t[n] x_t[n] + D_skip u_t
//   (naju/scan.py:79-93 of the reference project)
//
// One CTA owns a tile of TC time steps x 128 channels of one batch row; thread = channel,
// the N states of the channel live in registers.  The tile is staged once in shared memory
// (16-byte cp.async, coalesced) and walked twice:
//   pass 1  local scan from a zero state -> (P, S) = (product of f, chunk-end state)
//   carry   decoupled look-back over the preceding chunks of the same channel tile:
//           each chunk publishes its aggregate (P, S) and, once its own carry-in is known,
//           its inclusive state; a chunk folds aggregates backwards until it meets an
//           inclusive state.  Tiles are handed out by an atomic ticket in time-major order,
//           so every predecessor is already running; every wait is bounded.
//   pass 2  scan again from the true carry-in, emitting y.
// The inclusive chunk-end states double as the checkpoints the backward restarts from.
#include "common.cuh"
#include "params.h"

namespace naju {

template <typename TA, typename TG, int NS, int TC>
__global__ void __launch_bounds__(kThreads) fwd_simt_kernel(const FwdParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  TA* s_u = reinterpret_cast<TA*>(smem_raw);            // [TC][128]; reused for y
  TG* s_fl = reinterpret_cast<TG*>(s_u + TC * kDT);     // [TC][128]
  TG* s_il = s_fl + TC * kDT;                           // [TC][128]
  float* s_B = reinterpret_cast<float*>(s_il + TC * kDT);  // [TC][NS]
  float* s_C = s_B + TC * NS;                              // [TC][NS]
  __shared__ unsigned int s_ticket;

  const int tid = threadIdx.x;
  if (tid == 0) s_ticket = atomicAdd(&p.hdr->ticket, 1u);
  __syncthreads();
  const int64_t tile = s_ticket;
  const int per_chunk = p.B * p.ndt;
  const int c = static_cast<int>(tile / per_chunk);
  const int rem = static_cast<int>(tile % per_chunk);
  const int b = rem / p.ndt, dt = rem % p.ndt;
  if (c >= p.nchunks) {  // cannot happen with grid == ntiles; recorded instead of trusted
    if (tid == 0) atomicOr(&p.hdr->status, NAJU_ST_BAD_TILE);
    return;
  }
  const int t0 = c * TC;
  const int len = min(TC, p.T - t0);
  const int d0 = dt * kDT;
  const int cols = min(kDT, p.D - d0);
  const int d = d0 + tid;
  const bool d_ok = d < p.D;

  // ---- stage the tile
  load_tile_async(s_u, reinterpret_cast<const TA*>(p.u) + b * p.u_sb + t0 * p.u_st + d0, p.u_st,
                  len, cols, tid);
  load_tile_async(s_fl, reinterpret_cast<const TG*>(p.fl) + b * p.fl_sb + t0 * p.fl_st + d0,
                  p.fl_st, len, cols, tid);
  load_tile_async(s_il, reinterpret_cast<const TG*>(p.il) + b * p.il_sb + t0 * p.il_st + d0,
                  p.il_st, len, cols, tid);
  cp_async_commit();
  load_bc_tile<NS>(s_B, p.Bm, p.bc_dtype, b * p.bm_sb + t0 * p.bm_st, p.bm_st, len, p.N, tid);
  load_bc_tile<NS>(s_C, p.Cm, p.bc_dtype, b * p.cm_sb + t0 * p.cm_st, p.cm_st, len, p.N, tid);
  cp_async_wait_all();
  __syncthreads();

  // ---- pass 1: local scan from zero
  float x[NS];
#pragma unroll
  for (int n = 0; n < NS; ++n) x[n] = 0.f;
  float P = 1.f;
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

  // ---- carry-in by decoupled look-back
  const int64_t slot = tile * kDT + tid;
  float h[NS];
  float Pin = 1.f;  // product of f from t=0 up to the start of this chunk
  if (c == 0) {
#pragma unroll
    for (int n = 0; n < NS; ++n)
      h[n] = (p.h0 != nullptr && d_ok && n < p.N) ? p.h0[(static_cast<int64_t>(b) * p.D + d) * p.N + n] : 0.f;
  } else {
    p.aggP[slot] = P;
    float4* dstS = reinterpret_cast<float4*>(p.aggS + slot * NS);
#pragma unroll
    for (int q = 0; q < NS / 4; ++q)
      dstS[q] = make_float4(x[4 * q], x[4 * q + 1], x[4 * q + 2], x[4 * q + 3]);
    __threadfence();
    __syncthreads();
    if (tid == 0) st_release(p.flags + tile, 1);

    float accP = 1.f;
#pragma unroll
    for (int n = 0; n < NS; ++n) h[n] = 0.f;
    for (int j = c - 1; j >= 0; --j) {
      const int64_t jt = static_cast<int64_t>(j) * per_chunk + rem;
      const int64_t js = jt * kDT + tid;
      const int st = wait_flag(p.flags + jt);
      if (st == 0) {
        atomicOr(&p.hdr->status, NAJU_ST_LOOKBACK_TIMEOUT);
        break;
      }
      if (st == 2) {
        const float4* src = reinterpret_cast<const float4*>(p.ckS + js * NS);
#pragma unroll
        for (int q = 0; q < NS / 4; ++q) {
          const float4 v = __ldcg(src + q);
          h[4 * q + 0] = fmaf(accP, v.x, h[4 * q + 0]);
          h[4 * q + 1] = fmaf(accP, v.y, h[4 * q + 1]);
          h[4 * q + 2] = fmaf(accP, v.z, h[4 * q + 2]);
          h[4 * q + 3] = fmaf(accP, v.w, h[4 * q + 3]);
        }
        Pin = accP * __ldcg(p.ckP + js);
        break;
      }
      const float4* src = reinterpret_cast<const float4*>(p.aggS + js * NS);
#pragma unroll
      for (int q = 0; q < NS / 4; ++q) {
        const float4 v = __ldcg(src + q);
        h[4 * q + 0] = fmaf(accP, v.x, h[4 * q + 0]);
        h[4 * q + 1] = fmaf(accP, v.y, h[4 * q + 1]);
        h[4 * q + 2] = fmaf(accP, v.z, h[4 * q + 2]);
        h[4 * q + 3] = fmaf(accP, v.w, h[4 * q + 3]);
      }
      accP *= __ldcg(p.aggP + js);
    }
  }

  // ---- publish the inclusive chunk-end state (also the backward's checkpoint)
  {
    float4* dstS = reinterpret_cast<float4*>(p.ckS + slot * NS);
#pragma unroll
    for (int q = 0; q < NS / 4; ++q)
      dstS[q] = make_float4(fmaf(P, h[4 * q + 0], x[4 * q + 0]), fmaf(P, h[4 * q + 1], x[4 * q + 1]),
                            fmaf(P, h[4 * q + 2], x[4 * q + 2]), fmaf(P, h[4 * q + 3], x[4 * q + 3]));
    p.ckP[slot] = P * Pin;
    __threadfence();
    __syncthreads();
    if (tid == 0) st_release(p.flags + tile, 2);
  }

  // ---- pass 2: scan from the true carry-in, emit y into the u tile
  const float Dv = d_ok ? p.Dskip[d] : 0.f;
#pragma unroll
  for (int n = 0; n < NS; ++n) x[n] = h[n];
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
  if (c == p.nchunks - 1 && d_ok) {
    if (p.hT != nullptr) {
      float* o = p.hT + (static_cast<int64_t>(b) * p.D + d) * p.N;
#pragma unroll
      for (int n = 0; n < NS; ++n)
        if (n < p.N) o[n] = x[n];
    }
    if (p.pT != nullptr) p.pT[static_cast<int64_t>(b) * p.D + d] = P * Pin;
  }
  __syncthreads();
  store_tile(reinterpret_cast<TA*>(p.y) + (static_cast<int64_t>(b) * p.T + t0) * p.D + d0, s_u,
             static_cast<int64_t>(p.D), len, cols, tid);
}

template <typename TA, typename TG, int NS>
static int launch_ns(const FwdParams& p, const Geometry& g, cudaStream_t st) {
  constexpr int TC = (NS <= 32) ? 64 : 32;
  const size_t smem = static_cast<size_t>(TC) * kDT * (sizeof(TA) + 2 * sizeof(TG)) +
                      2 * static_cast<size_t>(TC) * NS * 4;
  auto kern = fwd_simt_kernel<TA, TG, NS, TC>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem));
  if (e != cudaSuccess) return static_cast<int>(e);
  kern<<<static_cast<unsigned>(g.ntiles), kThreads, smem, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}

template <typename TA, typename TG>
static int launch_types(const FwdParams& p, const Geometry& g, cudaStream_t st) {
  switch (g.NS) {
    case 16: return launch_ns<TA, TG, 16>(p, g, st);
    case 32: return launch_ns<TA, TG, 32>(p, g, st);
    case 64: return launch_ns<TA, TG, 64>(p, g, st);
    default: return launch_ns<TA, TG, 128>(p, g, st);
  }
}

int launch_fwd_simt(const FwdParams& p, const Geometry& g, int act, int gate, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (act == NAJU_F32 && gate == NAJU_F32) return launch_types<float, float>(p, g, st);
  if (act == NAJU_BF16 && gate == NAJU_BF16) return launch_types<__nv_bfloat16, __nv_bfloat16>(p, g, st);
  if (act == NAJU_BF16 && gate == NAJU_F32) return launch_types<__nv_bfloat16, float>(p, g, st);
  if (act == NAJU_F16 && gate == NAJU_F16) return launch_types<__half, __half>(p, g, st);
  if (act == NAJU_F16 && gate == NAJU_F32) return launch_types<__half, float>(p, g, st);
  return NAJU_E_DTYPE;
}

}  // namespace naju
