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
#include "fwd_common.cuh"

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
  if (tid == 0) {
    s_ticket = atomicAdd(&p.hdr->ticket, 1u);
    if (blockIdx.x == 0) p.hdr->form = NAJU_FORM_RECURRENT;
  }
  __syncthreads();
  TileCoord tc;
  if (!decode_tile<TC>(s_ticket, p.B, p.T, p.D, p.nchunks, p.ndt, tid, tc)) {
    if (tid == 0) atomicOr(&p.hdr->status, NAJU_ST_BAD_TILE);  // never expected
    return;
  }
  const int b = tc.b, t0 = tc.t0, len = tc.len, d0 = tc.d0, cols = tc.cols;

  // ---- stage the tile
  if (p.u_sd > 1)
    load_tile_tmajor(s_u, reinterpret_cast<const TA*>(p.u) + b * p.u_sb + t0 + d0 * p.u_sd, p.u_sd, len, cols, tid);
  else
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

  float x[NS], h[NS];
  float P, Pin;
  tile_pass1<TA, TG, NS>(s_u, s_fl, s_il, s_B, len, tid, x, P);
  carry_lookback<NS>(p, tc, tid, x, P, h, Pin);
  const float Dv = tc.d_ok ? p.Dskip[tc.d] : 0.f;
  tile_pass2<TA, TG, NS>(s_u, s_fl, s_il, s_B, s_C, len, tid, Dv, h);
  write_final<NS>(p, tc, h, P * Pin);
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
