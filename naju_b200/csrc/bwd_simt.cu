// Backward gated scan, exact recurrent form: every gradient in one reverse-time pass,
// without materialising the state history.
//
// Adjoint of naju/scan.py:79-93 as written out in naju/cuda/naju_cuda.cu:85-144:
//   xbar_t = dy_t C_t + f_{t+1} xbar_{t+1}
//   dC_t[n] = sum_d dy_t x_t[n]          dB_t[n] = sum_d xbar_t[n] w_t      (w = i u)
//   g_t = <xbar_t, B_t>   du_t = i_t g_t + D_skip dy_t   d i_logit_t = g_t w_t (1 - i_t)
//   d f_logit_t = (1 - f_t) r_t,  r_t = <xbar_t, x_t> - w_t g_t
// (the last line is the division-free form naju/chunk_bwd_triton.py:90-91 uses).
//
// r_t obeys a scalar recurrence, r_t = r_{t+1} + dy_t <C_t, x_t> - w_t g_t, seeded at the
// chunk end by r = <carry_in, x_end>.  That removes the need to hold x_t and xbar_t at the
// same time: a tile (TC steps x 128 channels, thread = channel) is walked once forward from
// the chunk-start state the forward saved (states, dC, dy*cx, the adjoint aggregate) and once
// in reverse (adjoint, dB, du, d f_logit, d i_logit).  The adjoint carry crosses chunks by the
// same bounded decoupled look-back as the forward, run towards later chunks.
// dB/dC are reduced over the tile's channels by a fixed-order warp reduce-scatter and written
// as per-channel-tile partials; small finalize kernels add the partials (deterministic).
#include "common.cuh"
#include "params.h"

#include <algorithm>

namespace naju {

constexpr int kG = 8;  // time steps between two cross-warp partial-sum flushes
// Below this retention the difference form of d f_logit loses more than ~3e-5 relative
// accuracy (it matches the f_logit >= -5 envelope of naju/chunk_triton.py:200).
constexpr float kDeepGate = 0.0078125f;

template <typename TA, typename TG, int NS, int TC>
__global__ void __launch_bounds__(kThreads) bwd_simt_kernel(const BwdParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  TA* s_u = reinterpret_cast<TA*>(smem_raw);             // [TC][128]; reused for du
  TA* s_dy = s_u + TC * kDT;                             // [TC][128]
  TG* s_fl = reinterpret_cast<TG*>(s_dy + TC * kDT);     // [TC][128]; reused for dfl
  TG* s_il = s_fl + TC * kDT;                            // [TC][128]; reused for dil
  float* s_B = reinterpret_cast<float*>(s_il + TC * kDT);   // [TC][NS]
  float* s_C = s_B + TC * NS;                               // [TC][NS]
  float* s_a = s_C + TC * NS;                               // [TC][128]  dy_t * <C_t, x_t>
  float* s_part = s_a + TC * kDT;                           // [kWarps][kG][NS]
  __shared__ unsigned int s_ticket;

  // the tensor-core backward was launched for this call and is doing the work
  if (p.tc_launched && (*p.fwd_form & 3) == 1) return;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (blockIdx.x == 0 && tid == 0) p.hdr->form = NAJU_FORM_RECURRENT;
  // Persistent CTAs: each takes tile tickets (reverse-time-major, so the chunk a tile waits on is
  // always held by a running CTA or done) until they run out.  The grid is a few CTAs per SM, which
  // also makes the stand-down above cost a few microseconds instead of one CTA launch per tile.
  for (;;) {
  __syncthreads();  // the previous tile is done with shared memory (and with s_ticket)
  if (tid == 0) s_ticket = atomicAdd(&p.hdr->ticket, 1u);
  __syncthreads();
  const int per_chunk = p.B * p.ndt;
  const int order = static_cast<int>(s_ticket / per_chunk);  // 0 = last chunk in time
  const int rem = static_cast<int>(s_ticket % per_chunk);
  if (order >= p.nchunks) return;
  const int c = p.nchunks - 1 - order;
  const int b = rem / p.ndt, dt = rem % p.ndt;
  const int64_t tile = static_cast<int64_t>(c) * per_chunk + rem;
  const int t0 = c * TC;
  const int len = min(TC, p.T - t0);
  const int d0 = dt * kDT;
  const int cols = min(kDT, p.D - d0);
  const int d = d0 + tid;
  const bool d_ok = d < p.D;

  if (p.u_sd > 1)
    load_tile_tmajor(s_u, reinterpret_cast<const TA*>(p.u) + b * p.u_sb + t0 + d0 * p.u_sd, p.u_sd, len, cols, tid);
  else
    load_tile_async(s_u, reinterpret_cast<const TA*>(p.u) + b * p.u_sb + t0 * p.u_st + d0, p.u_st,
                    len, cols, tid);
  load_tile_async(s_dy, reinterpret_cast<const TA*>(p.dy) + (static_cast<int64_t>(b) * p.T + t0) * p.D + d0,
                  static_cast<int64_t>(p.D), len, cols, tid);
  load_tile_async(s_fl, reinterpret_cast<const TG*>(p.fl) + b * p.fl_sb + t0 * p.fl_st + d0,
                  p.fl_st, len, cols, tid);
  load_tile_async(s_il, reinterpret_cast<const TG*>(p.il) + b * p.il_sb + t0 * p.il_st + d0,
                  p.il_st, len, cols, tid);
  cp_async_commit();
  load_bc_tile<NS>(s_B, p.Bm, p.bc_dtype, b * p.bm_sb + t0 * p.bm_st, p.bm_st, len, p.N, tid);
  load_bc_tile<NS>(s_C, p.Cm, p.bc_dtype, b * p.cm_sb + t0 * p.cm_st, p.cm_st, len, p.N, tid);

  // chunk-start state: the forward's inclusive state of the previous chunk (or h0)
  float x[NS];
  if (c == 0) {
#pragma unroll
    for (int n = 0; n < NS; ++n)
      x[n] = (p.h0 != nullptr && d_ok && n < p.N) ? p.h0[(static_cast<int64_t>(b) * p.D + d) * p.N + n] : 0.f;
  } else {
    const float4* src =
        reinterpret_cast<const float4*>(p.ckS + ((tile - per_chunk) * kDT + tid) * NS);
#pragma unroll
    for (int q = 0; q < NS / 4; ++q) {
      const float4 v = __ldg(src + q);
      x[4 * q] = v.x; x[4 * q + 1] = v.y; x[4 * q + 2] = v.z; x[4 * q + 3] = v.w;
    }
  }
  cp_async_wait_all();
  __syncthreads();

  const int nbase = WarpRS<NS>::out_base(lane);
  constexpr int OC = WarpRS<NS>::out_count;
  // For NS == 16 lanes 2k and 2k+1 end up with the same total; only even lanes write it.
  const bool writer = (NS >= 32) || ((lane & 1) == 0);
  const int64_t part_row0 = (static_cast<int64_t>(b) * p.T + t0) * p.ndt + dt;  // + t*ndt

  // ---------------- forward walk: states, dC partials, a_t, adjoint aggregate
  float lam[NS];
#pragma unroll
  for (int n = 0; n < NS; ++n) lam[n] = 0.f;
  float P = 1.f, dDsum = 0.f;
  for (int tg = 0; tg < len; tg += kG) {
#pragma unroll 1
    for (int g = 0; g < kG; ++g) {
      const int t = tg + g;
      if (t < len) {
        const float ut = to_f32(s_u[t * kDT + tid]);
        const float dyt = to_f32(s_dy[t * kDT + tid]);
        const float f = sigmoid_f(to_f32(s_fl[t * kDT + tid]));
        const float w = sigmoid_f(to_f32(s_il[t * kDT + tid])) * ut;
        P *= f;
        dDsum = fmaf(dyt, ut, dDsum);
        const float pdy = P * dyt;
        const float4* Bt = reinterpret_cast<const float4*>(s_B + t * NS);
        const float4* Ct = reinterpret_cast<const float4*>(s_C + t * NS);
        float cx = 0.f;
        float dc[NS];
#pragma unroll
        for (int q = 0; q < NS / 4; ++q) {
          const float4 bv = Bt[q];
          const float4 cv = Ct[q];
          x[4 * q + 0] = fmaf(f, x[4 * q + 0], w * bv.x);
          x[4 * q + 1] = fmaf(f, x[4 * q + 1], w * bv.y);
          x[4 * q + 2] = fmaf(f, x[4 * q + 2], w * bv.z);
          x[4 * q + 3] = fmaf(f, x[4 * q + 3], w * bv.w);
          cx = fmaf(cv.x, x[4 * q + 0], cx);
          cx = fmaf(cv.y, x[4 * q + 1], cx);
          cx = fmaf(cv.z, x[4 * q + 2], cx);
          cx = fmaf(cv.w, x[4 * q + 3], cx);
          lam[4 * q + 0] = fmaf(pdy, cv.x, lam[4 * q + 0]);
          lam[4 * q + 1] = fmaf(pdy, cv.y, lam[4 * q + 1]);
          lam[4 * q + 2] = fmaf(pdy, cv.z, lam[4 * q + 2]);
          lam[4 * q + 3] = fmaf(pdy, cv.w, lam[4 * q + 3]);
          dc[4 * q + 0] = dyt * x[4 * q + 0];
          dc[4 * q + 1] = dyt * x[4 * q + 1];
          dc[4 * q + 2] = dyt * x[4 * q + 2];
          dc[4 * q + 3] = dyt * x[4 * q + 3];
        }
        s_a[t * kDT + tid] = dyt * cx;
        WarpRS<NS>::run(dc, lane);
        if (writer) {
#pragma unroll
          for (int j = 0; j < OC; ++j) s_part[(warp * kG + g) * NS + nbase + j] = dc[j];
        }
      }
    }
    __syncthreads();
    for (int e = tid; e < kG * NS; e += kThreads) {
      const int g = e / NS, n = e % NS;
      if (tg + g < len) {
        float s = 0.f;
#pragma unroll
        for (int wq = 0; wq < kWarps; ++wq) s += s_part[(wq * kG + g) * NS + n];
        p.dCpart[(part_row0 + static_cast<int64_t>(tg + g) * p.ndt) * NS + n] = s;
      }
    }
    __syncthreads();
  }
  p.dDpart[(static_cast<int64_t>(c) * p.B + b) * (p.ndt * kDT) + d0 + tid] = dDsum;

  // ---------------- adjoint carry-in by decoupled look-back towards later chunks
  const int64_t slot = tile * kDT + tid;
  float carry[NS];
  if (c == p.nchunks - 1) {
#pragma unroll
    for (int n = 0; n < NS; ++n)
      carry[n] = (p.dhT != nullptr && d_ok && n < p.N) ? p.dhT[(static_cast<int64_t>(b) * p.D + d) * p.N + n] : 0.f;
  } else {
    p.aggP[slot] = P;
    float4* dstL = reinterpret_cast<float4*>(p.aggL + slot * NS);
#pragma unroll
    for (int q = 0; q < NS / 4; ++q)
      dstL[q] = make_float4(lam[4 * q], lam[4 * q + 1], lam[4 * q + 2], lam[4 * q + 3]);
    __threadfence();
    __syncthreads();
    if (tid == 0) st_release(p.flags + tile, 1);

    float accP = 1.f;
#pragma unroll
    for (int n = 0; n < NS; ++n) carry[n] = 0.f;
    for (int j = c + 1; j < p.nchunks; ++j) {
      const int64_t jt = static_cast<int64_t>(j) * per_chunk + rem;
      const int64_t js = jt * kDT + tid;
      const int st = wait_flag(p.flags + jt);
      if (st == 0) {
        atomicOr(&p.hdr->status, NAJU_ST_LOOKBACK_TIMEOUT);
        break;
      }
      const float4* src = reinterpret_cast<const float4*>((st == 2 ? p.inclL : p.aggL) + js * NS);
#pragma unroll
      for (int q = 0; q < NS / 4; ++q) {
        const float4 v = __ldcg(src + q);
        carry[4 * q + 0] = fmaf(accP, v.x, carry[4 * q + 0]);
        carry[4 * q + 1] = fmaf(accP, v.y, carry[4 * q + 1]);
        carry[4 * q + 2] = fmaf(accP, v.z, carry[4 * q + 2]);
        carry[4 * q + 3] = fmaf(accP, v.w, carry[4 * q + 3]);
      }
      if (st == 2) break;
      accP *= __ldcg(p.aggP + js);
    }
  }
  // inclusive adjoint leaving this chunk towards earlier time: lam + P * carry_in
  {
    float4* dstL = reinterpret_cast<float4*>(p.inclL + slot * NS);
#pragma unroll
    for (int q = 0; q < NS / 4; ++q)
      dstL[q] = make_float4(fmaf(P, carry[4 * q + 0], lam[4 * q + 0]), fmaf(P, carry[4 * q + 1], lam[4 * q + 1]),
                            fmaf(P, carry[4 * q + 2], lam[4 * q + 2]), fmaf(P, carry[4 * q + 3], lam[4 * q + 3]));
    __threadfence();
    __syncthreads();
    if (tid == 0) st_release(p.flags + tile, 2);
    if (c == 0 && p.dh0 != nullptr && d_ok) {
      float* o = p.dh0 + (static_cast<int64_t>(b) * p.D + d) * p.N;
#pragma unroll
      for (int n = 0; n < NS; ++n)
        if (n < p.N) o[n] = fmaf(P, carry[n], lam[n]);
    }
  }

  // ---------------- reverse walk
  float r = 0.f;
#pragma unroll
  for (int n = 0; n < NS; ++n) r = fmaf(carry[n], x[n], r);
  const float Dv = d_ok ? p.Dskip[d] : 0.f;
  const int last_group = ((len - 1) / kG) * kG;
  for (int tg = last_group; tg >= 0; tg -= kG) {
#pragma unroll 1
    for (int g = kG - 1; g >= 0; --g) {
      const int t = tg + g;
      if (t < len) {
        const float ut = to_f32(s_u[t * kDT + tid]);
        const float dyt = to_f32(s_dy[t * kDT + tid]);
        const Gate fg = gate(to_f32(s_fl[t * kDT + tid]));
        const Gate ig = gate(to_f32(s_il[t * kDT + tid]));
        const float f = fg.s, w = ig.s * ut;
        const float4* Bt = reinterpret_cast<const float4*>(s_B + t * NS);
        const float4* Ct = reinterpret_cast<const float4*>(s_C + t * NS);
        // Deep retention gate: r_t = f_t <xbar_t, x_{t-1}> is then far smaller than the two
        // terms whose difference the recurrence forms, so it is computed directly instead,
        // from x_{t-1} re-walked from the chunk-start state (rare; cost O(t) for this thread).
        const bool deep = f < kDeepGate;
        float r_exact = 0.f;
        if (deep) {
          float xp[NS];
          if (c == 0) {
#pragma unroll
            for (int n = 0; n < NS; ++n)
              xp[n] = (p.h0 != nullptr && d_ok && n < p.N) ? p.h0[(static_cast<int64_t>(b) * p.D + d) * p.N + n] : 0.f;
          } else {
            const float4* src =
                reinterpret_cast<const float4*>(p.ckS + ((tile - per_chunk) * kDT + tid) * NS);
#pragma unroll
            for (int q = 0; q < NS / 4; ++q) {
              const float4 v = __ldg(src + q);
              xp[4 * q] = v.x; xp[4 * q + 1] = v.y; xp[4 * q + 2] = v.z; xp[4 * q + 3] = v.w;
            }
          }
          for (int tt = 0; tt < t; ++tt) {  // inputs of steps < t are still intact in smem
            const float f2 = sigmoid_f(to_f32(s_fl[tt * kDT + tid]));
            const float w2 = sigmoid_f(to_f32(s_il[tt * kDT + tid])) * to_f32(s_u[tt * kDT + tid]);
            const float4* B2 = reinterpret_cast<const float4*>(s_B + tt * NS);
#pragma unroll
            for (int q = 0; q < NS / 4; ++q) {
              const float4 bv = B2[q];
              xp[4 * q + 0] = fmaf(f2, xp[4 * q + 0], w2 * bv.x);
              xp[4 * q + 1] = fmaf(f2, xp[4 * q + 1], w2 * bv.y);
              xp[4 * q + 2] = fmaf(f2, xp[4 * q + 2], w2 * bv.z);
              xp[4 * q + 3] = fmaf(f2, xp[4 * q + 3], w2 * bv.w);
            }
          }
          float dot = 0.f;
#pragma unroll
          for (int q = 0; q < NS / 4; ++q) {
            const float4 cv = Ct[q];
            dot = fmaf(fmaf(cv.x, dyt, carry[4 * q + 0]), xp[4 * q + 0], dot);
            dot = fmaf(fmaf(cv.y, dyt, carry[4 * q + 1]), xp[4 * q + 1], dot);
            dot = fmaf(fmaf(cv.z, dyt, carry[4 * q + 2]), xp[4 * q + 2], dot);
            dot = fmaf(fmaf(cv.w, dyt, carry[4 * q + 3]), xp[4 * q + 3], dot);
          }
          r_exact = f * dot;
        }
        float gsum = 0.f;
        float db[NS];
#pragma unroll
        for (int q = 0; q < NS / 4; ++q) {
          const float4 bv = Bt[q];
          const float4 cv = Ct[q];
          const float dx0 = fmaf(cv.x, dyt, carry[4 * q + 0]);
          const float dx1 = fmaf(cv.y, dyt, carry[4 * q + 1]);
          const float dx2 = fmaf(cv.z, dyt, carry[4 * q + 2]);
          const float dx3 = fmaf(cv.w, dyt, carry[4 * q + 3]);
          gsum = fmaf(dx0, bv.x, gsum);
          gsum = fmaf(dx1, bv.y, gsum);
          gsum = fmaf(dx2, bv.z, gsum);
          gsum = fmaf(dx3, bv.w, gsum);
          db[4 * q + 0] = dx0 * w; db[4 * q + 1] = dx1 * w;
          db[4 * q + 2] = dx2 * w; db[4 * q + 3] = dx3 * w;
          carry[4 * q + 0] = f * dx0; carry[4 * q + 1] = f * dx1;
          carry[4 * q + 2] = f * dx2; carry[4 * q + 3] = f * dx3;
        }
        r += s_a[t * kDT + tid] - w * gsum;
        if (deep) r = r_exact;
        s_u[t * kDT + tid] = from_f32<TA>(fmaf(ig.s, gsum, Dv * dyt));
        s_fl[t * kDT + tid] = from_f32<TG>(fg.one_minus * r);
        s_il[t * kDT + tid] = from_f32<TG>(gsum * w * ig.one_minus);
        WarpRS<NS>::run(db, lane);
        if (writer) {
#pragma unroll
          for (int j = 0; j < OC; ++j) s_part[(warp * kG + g) * NS + nbase + j] = db[j];
        }
      }
    }
    __syncthreads();
    for (int e = tid; e < kG * NS; e += kThreads) {
      const int g = e / NS, n = e % NS;
      if (tg + g < len) {
        float s = 0.f;
#pragma unroll
        for (int wq = 0; wq < kWarps; ++wq) s += s_part[(wq * kG + g) * NS + n];
        p.dBpart[(part_row0 + static_cast<int64_t>(tg + g) * p.ndt) * NS + n] = s;
      }
    }
    __syncthreads();
  }

  const int64_t out_off = (static_cast<int64_t>(b) * p.T + t0) * p.D + d0;
  if (p.u_sd > 1)   // du in the layout of a time-contiguous u
    store_tile_tmajor(reinterpret_cast<TA*>(p.du) + b * p.u_sb + t0 + d0 * p.u_sd, s_u, p.u_sd, len, cols, tid);
  else
    store_tile(reinterpret_cast<TA*>(p.du) + out_off, s_u, static_cast<int64_t>(p.D), len, cols, tid);
  store_tile(reinterpret_cast<TG*>(p.dfl) + out_off, s_fl, static_cast<int64_t>(p.D), len, cols, tid);
  store_tile(reinterpret_cast<TG*>(p.dil) + out_off, s_il, static_cast<int64_t>(p.D), len, cols, tid);
  }
}

// out[row][n] = sum_k part[row][k][n] for n < N, written in the caller's dtype
__global__ void finalize_bc_kernel(const float* __restrict__ part, void* __restrict__ out,
                                   int64_t rows, int ndt, int NS, int N, int dtype) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= rows * N) return;
  const int64_t row = i / N;
  const int n = static_cast<int>(i % N);
  float s = 0.f;
  for (int k = 0; k < ndt; ++k) s += part[(row * ndt + k) * NS + n];
  store_dyn(out, dtype, i, s);
}

// dD[d] = sum_rows part[row][d]; block = 32 channels x 32 row lanes, fixed-order tree
__global__ void finalize_dD_kernel(const float* __restrict__ part, float* __restrict__ dD,
                                   int rows, int rows_tc, const int* __restrict__ fwd_form, int ld, int D) {
  __shared__ float red[32][33];
  // the tensor-core backward writes two partial rows per batch row, the recurrent one per chunk
  if (rows_tc > 0 && (*fwd_form & 3) == 1) rows = rows_tc;
  const int dl = threadIdx.x, rl = threadIdx.y;
  const int d = blockIdx.x * 32 + dl;
  float s = 0.f;
  if (d < D)
    for (int r = rl; r < rows; r += 32) s += part[static_cast<int64_t>(r) * ld + d];
  red[rl][dl] = s;
  __syncthreads();
  if (rl == 0 && d < D) {
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < 32; ++k) tot += red[k][dl];
    dD[d] = tot;
  }
}

template <typename TA, typename TG, int NS>
static int launch_ns(const BwdParams& p, const Geometry& g, cudaStream_t st) {
  constexpr int TC = (NS <= 32) ? 64 : 32;
  const size_t smem = static_cast<size_t>(TC) * kDT * (2 * sizeof(TA) + 2 * sizeof(TG)) +
                      2 * static_cast<size_t>(TC) * NS * 4 + static_cast<size_t>(TC) * kDT * 4 +
                      static_cast<size_t>(kWarps) * kG * NS * 4;
  auto kern = bwd_simt_kernel<TA, TG, NS, TC>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem));
  if (e != cudaSuccess) return static_cast<int>(e);
  // persistent grid: what fits on the GPU at once (the look-back needs every waiting CTA's
  // predecessors to be resident or done, which ticket order guarantees for any grid size)
  int dev = 0, sms = 148, per_sm = 1;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThreads, smem) != cudaSuccess || per_sm < 1)
    per_sm = 1;
  const int64_t grid = std::min<int64_t>(g.ntiles, static_cast<int64_t>(sms) * per_sm);
  kern<<<static_cast<unsigned>(grid), kThreads, smem, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}

template <typename TA, typename TG>
static int launch_types(const BwdParams& p, const Geometry& g, cudaStream_t st) {
  switch (g.NS) {
    case 16: return launch_ns<TA, TG, 16>(p, g, st);
    case 32: return launch_ns<TA, TG, 32>(p, g, st);
    case 64: return launch_ns<TA, TG, 64>(p, g, st);
    default: return launch_ns<TA, TG, 128>(p, g, st);
  }
}

int launch_bwd_simt(const BwdParams& p, const Geometry& g, int act, int gate, void* dB, void* dC,
                    float* dD, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc;
  if (act == NAJU_F32 && gate == NAJU_F32) rc = launch_types<float, float>(p, g, st);
  else if (act == NAJU_BF16 && gate == NAJU_BF16) rc = launch_types<__nv_bfloat16, __nv_bfloat16>(p, g, st);
  else if (act == NAJU_BF16 && gate == NAJU_F32) rc = launch_types<__nv_bfloat16, float>(p, g, st);
  else if (act == NAJU_F16 && gate == NAJU_F16) rc = launch_types<__half, __half>(p, g, st);
  else if (act == NAJU_F16 && gate == NAJU_F32) rc = launch_types<__half, float>(p, g, st);
  else return NAJU_E_DTYPE;
  if (rc != 0) return rc;

  const int64_t rows = static_cast<int64_t>(g.B) * g.T;
  const int64_t total = rows * g.N;
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
  finalize_bc_kernel<<<blocks, 256, 0, st>>>(p.dBpart, dB, rows, g.ndt, g.NS, g.N, p.bc_dtype);
  finalize_bc_kernel<<<blocks, 256, 0, st>>>(p.dCpart, dC, rows, g.ndt, g.NS, g.N, p.bc_dtype);
  finalize_dD_kernel<<<(g.D + 31) / 32, dim3(32, 32), 0, st>>>(p.dDpart, dD, g.nchunks * g.B,
                                                              p.tc_launched ? 4 * g.B : 0, p.fwd_form,
                                                              g.ndt * kDT, g.D);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace naju
