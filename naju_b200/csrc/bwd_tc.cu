// Backward gated scan, chunked (state-expansion) form on tcgen05 tensor cores.
//
// A CTA owns channel tiles (one batch row x 128 channels; one per CTA, or dealt round-robin when
// there are more tiles than SMs) and walks each one's chunks of Q = 64 steps in REVERSE time; the
// adjoint carry stays in registers, the state entering each chunk comes from the checkpoints the
// forward saved.  Per chunk and channel d, with P_t = prod f,
// R_t = 1/P_t, wt_s = w_s R_s (w = sigmoid(i_logit) u), al_t = dy_t P_t, h the state entering
// the chunk, lam the adjoint entering it from the future, lt = P_Q lam and G = tril(C B^T):
//
//   Yt[d,t] = sum_{s<=t} G[t,s] wt[d,s] + <C_t, h[d]>            (forward readout / P_t)
//   gt[d,s] = sum_{t>=s} G[t,s] al[d,t] + <B_s, lt[d]>           (g_s / R_s, g = <xbar, B>)
//   dL[d,n] = sum_t al[d,t] C[t,n]                               (adjoint leaving the chunk - P_Q lam)
//   M2[t,s] = sum_d al[d,t] wt[d,s],  U[t,n] = sum_d al[d,t] h[d,n],  V[s,n] = sum_d wt[d,s] lt[d,n]
//   dC[t,n] = U[t,n] + sum_{s<=t} M2[t,s] B[s,n]      dB[s,n] = V[s,n] + sum_{t>=s} M2[t,s] C[t,n]
//
// (the adjoint of naju/scan.py:79-93 as written out in naju/cuda/naju_cuda.cu:85-144; the Gram
// form of dB/dC is the one naju/chunk_bwd_triton.py:20-99 uses on 16-step blocks).  Then
//   r_t = r_{t+1} + al_t Yt_t - wt_t gt_t  (r at the chunk end = <lam, x_end>),
//   d f_logit = (1-f_t) r_t,  du = (i_t R_t) gt_t + D_skip dy_t,  d i_logit = wt_t (1-i_t) gt_t.
// All seven contractions are tcgen05.mma (kind::f16, bf16 operands in two-term splits, fp32
// accumulators in TMEM, M = 128).  Each channel owns one row [al | wt | h | lt] in shared memory;
// the same bytes serve as K-major operands for the per-channel GEMMs (contraction over time or
// state) and as MN-major operands for the cross-channel ones (contraction over the 128 channels),
// and the G buffer serves K-major for Yt and MN-major (i.e. transposed) for gt.
//
// Warps: 0-7 main, two threads per channel (gates -> operand rows and per-step coefficients into
// TMEM; after the MMAs the reverse-time sweep; the output tiles leave by TMA store), 8 TMA
// producer, 9 shared-operand builder (mma.sync), 10 MMA issuer.  Every wait is bounded.  Tiles with deep retention gates (prod f < 2^-80 in a
// chunk) cannot be factorised; the forward records whether it met one, and this kernel stands
// down in that case (the exact recurrent backward runs instead).
#include <algorithm>
#include <type_traits>

#include "common.cuh"
#include "params.h"
#include "tc_common.cuh"
#include "tma_host.h"

namespace naju {
namespace tcb {

using namespace tcx;

constexpr int Q = 64, NS = 16, SLAB = 16, NSLAB = Q / SLAB, RING = 4;
constexpr int NMAIN = 256, NHALF = 128, NTHREADS = 352;
// channel row (bf16, chunks of 8): [al1 8 | w1 8 | h1 2 | l1 2 | al2 8 | w2 8 | h2 2 | l2 2]
constexpr int R_A1 = 0, R_W1 = 8, R_H1 = 16, R_L1 = 18, R_A2 = 20, R_W2 = 28, R_H2 = 36, R_L2 = 38, R_CH = 40;
constexpr uint32_t SBO_R = R_CH * 128, ROWS_BYTES = 16 * SBO_R;  // 81920
// BG rows t: [C 2 | g1 8 | g2 8]
constexpr int BG_C = 0, BG_G1 = 2, BG_G2 = 10;
constexpr uint32_t SBO_BG = 18 * 128, BG_BYTES = 8 * SBO_BG;     // 18432
constexpr uint32_t SBO_BB = 2 * 128, BB_BYTES = 8 * SBO_BB;      // rows s: [B 2]        2048
constexpr uint32_t SBO_T = 8 * 128, T_BYTES = 2 * SBO_T;         // rows n: [X^T 8]      2048 (CT and BT)
// M2 operand rows t: [m1 8 | m2 8]; 64 real rows, addressed as 128 (the rest is never used)
constexpr int M_1 = 0, M_2 = 8;
constexpr uint32_t SBO_M = 16 * 128;                         // 8 row groups = 16384 bytes
constexpr uint32_t BC_BYTES = Q * NS * 2;
// TMEM columns
constexpr uint32_t TM_Y = 0, TM_G = 64, TM_DL = 128, TM_X = 144, TM_DCI = 240, TM_CF = 256, TM_CI = 320,
                   TM_CU = 384, TM_DBI = 448, TMEM_COLS = 512;
constexpr float kRMax = 1.0e24f;
constexpr float kNegLog2e = -1.4426950408889634f;

__device__ __forceinline__ float fast_ex2(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float fast_rcp(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// MN-major no-swizzle descriptor: `kgroup` = bytes between groups of 8 along K (LBO field),
// `mnchunk` = bytes between 8-element chunks along M/N (SBO field).
__device__ __forceinline__ uint64_t umma_desc_mn(uint32_t saddr, uint32_t kgroup, uint32_t mnchunk) {
  return umma_desc(saddr, kgroup, mnchunk);
}
__device__ __forceinline__ uint32_t idesc_bf16(int N, uint32_t a_mn, uint32_t b_mn) {
  return umma_idesc(128, N, 1) | (a_mn << 15) | (b_mn << 16);
}

#ifdef NAJU_PROF
__device__ unsigned long long g_profb[16];
#define PROFB_MARK(i)                                                      \
  do {                                                                     \
    if (tid == 0) {                                                        \
      const long long now_ = clock64();                                    \
      atomicAdd(&g_profb[i], static_cast<unsigned long long>(now_ - pt_)); \
      pt_ = now_;                                                          \
    }                                                                      \
  } while (0)
#define PROFB_INIT long long pt_ = clock64()
#else
#define PROFB_MARK(i) do {} while (0)
#define PROFB_INIT do {} while (0)
#endif

struct Maps {
  CUtensorMap u, fl, il, dy, bm, cm, du, dfl, dil;
};

// TG = type of the logits and of their gradients.  With 16-bit logits all three output tiles are
// staged in shared memory and written by TMA stores; with fp32 logits the input slabs are
// larger, only du is staged, and d f_logit / d i_logit go out straight from registers (a warp's
// 32 consecutive fp32 values are a full 128-byte line).
template <typename TG>
struct SmemT {
  static constexpr bool kStageGates = sizeof(TG) == 2;
  static constexpr uint32_t off_sfl = SLAB * kDT * 2;                       // slab: u | fl | il | dy
  static constexpr uint32_t off_sil = off_sfl + SLAB * kDT * sizeof(TG);
  static constexpr uint32_t off_sdy = off_sil + SLAB * kDT * sizeof(TG);
  static constexpr uint32_t slab_bytes = off_sdy + SLAB * kDT * 2;
  static constexpr uint32_t off_ring = 0;
  static constexpr uint32_t off_rows = off_ring + RING * slab_bytes;
  static constexpr uint32_t off_out = off_rows + ROWS_BYTES;      // du | dfl | dil staging, [64][128] each
  // The M2 operand re-uses the du staging tile: it is written after the staged outputs have been
  // stored and consumed (second MMA round) before the next sweep stages anything.  As an MMA
  // operand it is addressed as 128 rows (32 KB) although only 64 exist, so at least 16 KB of
  // shared memory must follow it: the staging tiles come before the shared operand buffers.
  static constexpr uint32_t off_M = off_out;
  static constexpr uint32_t off_BG = off_out + (kStageGates ? 3 : 1) * Q * kDT * 2;
  static constexpr uint32_t off_BB = off_BG + BG_BYTES;
  static constexpr uint32_t off_CT = off_BB + BB_BYTES;
  static constexpr uint32_t off_BT = off_CT + T_BYTES;
  static constexpr uint32_t off_bc = off_BT + T_BYTES;            // [2 tiles][B raw | C raw]
  static constexpr uint32_t total = off_bc + 2 * 2 * BC_BYTES;
  static_assert(off_M + 16 * SBO_M <= total, "the 128-row view of the M2 operand must stay inside shared memory");
};

struct Bars {
  unsigned long long full[RING], empty[RING];
  unsigned long long bc_full[2], bc_empty[2];
  unsigned long long part[NSLAB];  // operand-row chunks of one 16-step slab written (128 threads)
  unsigned long long carry_full;   // h and lt rows written
  unsigned long long opsA_full;    // C | g1 | g2 and B rows built (first MMA round, contraction over time/state)
  unsigned long long opsB_full;    // C^T and B^T built (dL and the second MMA round)
  unsigned long long d1_full, d4_full, m2_full, d5_full;
};

// MULTI: a CTA may be dealt more than one channel tile (grid = number of SMs); without it the grid is
// the number of channel tiles and the outer loops below run exactly once, which the compiler
// knows (the single-tile kernel needs a few registers less and does not spill).
template <typename TA, typename TG, bool MULTI>
__global__ void __launch_bounds__(NTHREADS, 1)
bwd_tc_kernel(const BwdParams p, const __grid_constant__ Maps maps, const int* __restrict__ fwd_form) {
  using Smem = SmemT<TG>;
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ Bars bars;
  __shared__ unsigned int s_tmem;
  __shared__ float s_PQ[kDT];  // chunk retention product per channel (second-half threads -> first-half)

  // stand down unless the forward ran in the chunked form and met no deep-gate tile
  if ((*fwd_form & 3) != 1) return;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t sbase = smem_u32(smem);
  // channel tiles (one batch row x 128 channels) are dealt round-robin over the grid; `it` counts
  // the (channel tile, chunk) pairs a CTA has seen and selects the barrier phases
  const int per_chunk = p.B * p.ndt;
  const int x_first = static_cast<int>(blockIdx.x), x_step = static_cast<int>(gridDim.x);
  const int nchunks = p.nchunks;

  if (tid == 0) {
    if (blockIdx.x == 0) p.hdr->form = NAJU_FORM_TC_WALK;
    for (int i = 0; i < RING; ++i) {
      mbar_init(smem_u32(&bars.full[i]), 1);
      mbar_init(smem_u32(&bars.empty[i]), NMAIN);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars.bc_full[i]), 1);
      mbar_init(smem_u32(&bars.bc_empty[i]), 1);
    }
    for (int i = 0; i < NSLAB; ++i) mbar_init(smem_u32(&bars.part[i]), NHALF);
    mbar_init(smem_u32(&bars.carry_full), NMAIN);
    mbar_init(smem_u32(&bars.opsA_full), 1);
    mbar_init(smem_u32(&bars.opsB_full), 1);
    mbar_init(smem_u32(&bars.d1_full), 1);
    mbar_init(smem_u32(&bars.d4_full), 1);
    mbar_init(smem_u32(&bars.m2_full), NMAIN);
    mbar_init(smem_u32(&bars.d5_full), 1);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(smem_u32(&s_tmem), TMEM_COLS);
  // zero the shared operand buffers once: the upper triangle of g1/g2 is never written afterwards
  for (uint32_t i = tid * 16; i < Smem::off_bc - Smem::off_BG; i += NTHREADS * 16)
    *reinterpret_cast<uint4*>(smem + Smem::off_BG + i) = make_uint4(0, 0, 0, 0);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;
  auto timeout = [&]() { atomicOr(&p.hdr->status, NAJU_ST_MMA_TIMEOUT); };

  if (warp == 8) {
    // ===================================================================== TMA producer
    if (lane == 0) {
      uint32_t slab = 0;
      int it = 0;
      int x = x_first;
      do {
      const int b = x / p.ndt, d0 = (x - b * p.ndt) * kDT;
      for (int ci = 0; ci < nchunks; ++ci, ++it) {
        const int c = nchunks - 1 - ci, t0 = c * Q, par = it & 1;
        if (it >= 2 && !mbar_wait(smem_u32(&bars.bc_empty[par]), ((it >> 1) & 1) ^ 1)) timeout();
        {
          const uint32_t bar = smem_u32(&bars.bc_full[par]);
          const uint32_t dst = sbase + Smem::off_bc + par * 2 * BC_BYTES;
          mbar_arrive_expect_tx(bar, 2 * BC_BYTES);
          tma_load_3d(dst, &maps.bm, 0, t0, b, bar);
          tma_load_3d(dst + BC_BYTES, &maps.cm, 0, t0, b, bar);
        }
        for (int k = 0; k < NSLAB; ++k, ++slab) {
          const uint32_t slot = slab % RING, ph = (slab / RING) & 1;
          if (slab >= RING && !mbar_wait(smem_u32(&bars.empty[slot]), ph ^ 1)) timeout();
          const uint32_t bar = smem_u32(&bars.full[slot]);
          const uint32_t dst = sbase + Smem::off_ring + slot * Smem::slab_bytes;
          mbar_arrive_expect_tx(bar, Smem::slab_bytes);
          tma_load_3d(dst, &maps.u, d0, t0 + k * SLAB, b, bar);
          tma_load_3d(dst + Smem::off_sfl, &maps.fl, d0, t0 + k * SLAB, b, bar);
          tma_load_3d(dst + Smem::off_sil, &maps.il, d0, t0 + k * SLAB, b, bar);
          tma_load_3d(dst + Smem::off_sdy, &maps.dy, d0, t0 + k * SLAB, b, bar);
        }
      }
      x += x_step;
      } while (MULTI && x < per_chunk);
    }
  } else if (warp == 9) {
    // ===================================================================== operand builder
    const int g = lane >> 2, t4 = lane & 3;
    unsigned char* s_BG = smem + Smem::off_BG;
    unsigned char* s_BB = smem + Smem::off_BB;
    unsigned char* s_CT = smem + Smem::off_CT;
    unsigned char* s_BT = smem + Smem::off_BT;
    const int ntile = MULTI ? ((per_chunk - x_first + x_step - 1) / x_step) * nchunks : nchunks;
    for (int it = 0; it < ntile; ++it) {
      const int par = it & 1;
      if (!mbar_wait(smem_u32(&bars.bc_full[par]), (it >> 1) & 1)) timeout();
      // C | g1 | g2 and the B rows are read only by the previous tile's first MMA round: they can
      // be rebuilt as soon as that round is complete, while the previous tile is still in its sweep
      if (it >= 1 && !mbar_wait(smem_u32(&bars.d1_full), (it - 1) & 1)) timeout();
      const __nv_bfloat16* Braw = reinterpret_cast<const __nv_bfloat16*>(smem + Smem::off_bc + par * 2 * BC_BYTES);
      const __nv_bfloat16* Craw = Braw + Q * NS;
      for (int e = lane; e < Q * 2; e += 32) {  // C into BG, B into BB: rows of 32 bytes
        const int t = e >> 1, half = e & 1;
        *reinterpret_cast<uint4*>(s_BG + op_off16(t, BG_C * 8 + half * 8, SBO_BG)) =
            *reinterpret_cast<const uint4*>(Craw + t * NS + half * 8);
        *reinterpret_cast<uint4*>(s_BB + op_off16(t, half * 8, SBO_BB)) =
            *reinterpret_cast<const uint4*>(Braw + t * NS + half * 8);
      }
#pragma unroll 1
      for (int mt = 0; mt < Q / 16; ++mt) {  // G = tril(C B^T), two bf16 terms
        const int r0 = 16 * mt + g, r1 = r0 + 8;
        const uint32_t a0 = *reinterpret_cast<const uint32_t*>(Craw + r0 * NS + 2 * t4);
        const uint32_t a1 = *reinterpret_cast<const uint32_t*>(Craw + r1 * NS + 2 * t4);
        const uint32_t a2 = *reinterpret_cast<const uint32_t*>(Craw + r0 * NS + 2 * t4 + 8);
        const uint32_t a3 = *reinterpret_cast<const uint32_t*>(Craw + r1 * NS + 2 * t4 + 8);
        for (int nt = 0; nt <= 2 * mt + 1; ++nt) {
          float c[4] = {0.f, 0.f, 0.f, 0.f};
          const uint32_t b0 = *reinterpret_cast<const uint32_t*>(Braw + (8 * nt + g) * NS + 2 * t4);
          const uint32_t b1 = *reinterpret_cast<const uint32_t*>(Braw + (8 * nt + g) * NS + 2 * t4 + 8);
          mma_bf16_16x8x16(c, a0, a1, a2, a3, b0, b1);
          const int s0 = 8 * nt + 2 * t4;
          uint32_t hi, lo;
          split_bf16x2(s0 <= r0 ? c[0] : 0.f, s0 + 1 <= r0 ? c[1] : 0.f, hi, lo);
          *reinterpret_cast<uint32_t*>(s_BG + op_off16(r0, BG_G1 * 8 + s0, SBO_BG)) = hi;
          *reinterpret_cast<uint32_t*>(s_BG + op_off16(r0, BG_G2 * 8 + s0, SBO_BG)) = lo;
          split_bf16x2(s0 <= r1 ? c[2] : 0.f, s0 + 1 <= r1 ? c[3] : 0.f, hi, lo);
          *reinterpret_cast<uint32_t*>(s_BG + op_off16(r1, BG_G1 * 8 + s0, SBO_BG)) = hi;
          *reinterpret_cast<uint32_t*>(s_BG + op_off16(r1, BG_G2 * 8 + s0, SBO_BG)) = lo;
        }
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars.opsA_full));
      // C^T and B^T are still read by the previous tile's second MMA round
      if (it >= 1 && !mbar_wait(smem_u32(&bars.d5_full), (it - 1) & 1)) timeout();
      for (int e = lane; e < NS * (Q / 8); e += 32) {  // C^T and B^T: (row n, eight columns t)
        const int n = e % NS, s8 = e / NS;
        uint32_t wc[4], wb[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int r0 = (8 * s8 + 2 * j) * NS + n, r1 = r0 + NS;
          wc[j] = static_cast<uint32_t>(reinterpret_cast<const unsigned short*>(Craw)[r0]) |
                  (static_cast<uint32_t>(reinterpret_cast<const unsigned short*>(Craw)[r1]) << 16);
          wb[j] = static_cast<uint32_t>(reinterpret_cast<const unsigned short*>(Braw)[r0]) |
                  (static_cast<uint32_t>(reinterpret_cast<const unsigned short*>(Braw)[r1]) << 16);
        }
        *reinterpret_cast<uint4*>(s_CT + op_off16(n, 8 * s8, SBO_T)) = make_uint4(wc[0], wc[1], wc[2], wc[3]);
        *reinterpret_cast<uint4*>(s_BT + op_off16(n, 8 * s8, SBO_T)) = make_uint4(wb[0], wb[1], wb[2], wb[3]);
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(&bars.opsB_full));
        mbar_arrive(smem_u32(&bars.bc_empty[par]));
      }
    }
  } else if (warp == 10) {
    // ===================================================================== MMA issuer
    if (lane == 0) {
      const uint32_t aR = sbase + Smem::off_rows, aBG = sbase + Smem::off_BG, aBB = sbase + Smem::off_BB;
      const uint32_t aCT = sbase + Smem::off_CT, aBT = sbase + Smem::off_BT, aM = sbase + Smem::off_M;
      const uint32_t iKK64 = idesc_bf16(64, 0, 0), iKM64 = idesc_bf16(64, 0, 1), iKK16 = idesc_bf16(16, 0, 0);
      const uint32_t iMM96 = idesc_bf16(96, 1, 1), iMK16 = idesc_bf16(16, 1, 0);
      // Every operand address is fixed, so the descriptors are built once; a descriptor for another
      // chunk / row group is the base plus (byte offset >> 4) in its address field.
      const uint64_t dRk = umma_desc(aR, 128, SBO_R), dRm = umma_desc(aR, SBO_R, 128);     // channel rows
      const uint64_t dGk = umma_desc(aBG, 128, SBO_BG), dGm = umma_desc(aBG, SBO_BG, 128);  // C | g1 | g2
      const uint64_t dBB = umma_desc(aBB, 128, SBO_BB), dCT = umma_desc(aCT, 128, SBO_T), dBT = umma_desc(aBT, 128, SBO_T);
      // M2 operand: K-major as is; MN-major starting eight chunks early, so that column s lands in
      // accumulator row 64+s (the lane of the thread that holds V[s,:]); rows 0-63 are never read
      const uint64_t dMk = umma_desc(aM, 128, SBO_M), dMm = umma_desc(aM - 8 * 128, SBO_M, 128);
      auto off = [](uint32_t bytes) { return static_cast<uint64_t>(bytes >> 4); };
      const int ntile = MULTI ? ((per_chunk - x_first + x_step - 1) / x_step) * nchunks : nchunks;
      for (int it = 0; it < ntile; ++it) {
        const uint32_t par = it & 1;
#ifdef NAJU_PROF
        const long long t_oa = clock64();
#endif
        if (!mbar_wait(smem_u32(&bars.opsA_full), par)) timeout();
#ifdef NAJU_PROF
        atomicAdd(&g_profb[14], static_cast<unsigned long long>(clock64() - t_oa));
#endif
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          // the MMAs that contract over time need only the row chunks of slab ks: they run while
          // the main warps are still evaluating the gates of the other slabs
#ifdef NAJU_PROF
          const long long t_p = clock64();
#endif
          if (!mbar_wait(smem_u32(&bars.part[ks]), par)) timeout();
#ifdef NAJU_PROF
          atomicAdd(&g_profb[12 + (ks >> 1)], static_cast<unsigned long long>(clock64() - t_p));
#endif
          tc_fence_after();
          // Yt += w1.g1 + w1.g2 + w2.g1   (K = s)
          const uint64_t g1 = dGk + off((BG_G1 + 2 * ks) * 128), g2 = dGk + off((BG_G2 + 2 * ks) * 128);
          umma_bf16(tmem + TM_Y, dRk + off((R_W1 + 2 * ks) * 128), g1, iKK64, ks > 0);
          umma_bf16(tmem + TM_Y, dRk + off((R_W1 + 2 * ks) * 128), g2, iKK64, 1u);
          umma_bf16(tmem + TM_Y, dRk + off((R_W2 + 2 * ks) * 128), g1, iKK64, 1u);
          if (ks == 0) {
            // Yt += (h1 + h2).C   (K = n): the h rows were written by the threads of slab 0 before
            // they released it, so this part of the carry does not have to wait for the carry barrier
            umma_bf16(tmem + TM_Y, dRk + off(R_H1 * 128), dGk + off(BG_C * 128), iKK64, 1u);
            umma_bf16(tmem + TM_Y, dRk + off(R_H2 * 128), dGk + off(BG_C * 128), iKK64, 1u);
          }
          // gt += al1.g1^T + al1.g2^T + al2.g1^T   (K = t: the G buffer read MN-major)
          const uint64_t g1t = dGm + off(2 * ks * SBO_BG + BG_G1 * 128), g2t = dGm + off(2 * ks * SBO_BG + BG_G2 * 128);
          umma_bf16(tmem + TM_G, dRk + off((R_A1 + 2 * ks) * 128), g1t, iKM64, ks > 0);
          umma_bf16(tmem + TM_G, dRk + off((R_A1 + 2 * ks) * 128), g2t, iKM64, 1u);
          umma_bf16(tmem + TM_G, dRk + off((R_A2 + 2 * ks) * 128), g1t, iKM64, 1u);
          // dL += al1.C + al2.C   (K = t, B operand = C^T rows), slab by slab as well; C^T comes a
          // little later than the other shared operands, so the first slab's share waits for ks = 1
          if (ks == 1) {
#ifdef NAJU_PROF
            const long long t_ob = clock64();
#endif
            if (!mbar_wait(smem_u32(&bars.opsB_full), par)) timeout();
#ifdef NAJU_PROF
            atomicAdd(&g_profb[15], static_cast<unsigned long long>(clock64() - t_ob));
#endif
            tc_fence_after();
            umma_bf16(tmem + TM_DL, dRk + off(R_A1 * 128), dCT, iKK16, 0u);
            umma_bf16(tmem + TM_DL, dRk + off(R_A2 * 128), dCT, iKK16, 1u);
          }
          if (ks >= 1) {
            umma_bf16(tmem + TM_DL, dRk + off((R_A1 + 2 * ks) * 128), dCT + off(2 * ks * 128), iKK16, 1u);
            umma_bf16(tmem + TM_DL, dRk + off((R_A2 + 2 * ks) * 128), dCT + off(2 * ks * 128), iKK16, 1u);
          }
        }
        // gt += (l1 + l2).B   (K = n): the only MMAs that need the whole chunk's retention product
        if (!mbar_wait(smem_u32(&bars.carry_full), par)) timeout();
        tc_fence_after();
        umma_bf16(tmem + TM_G, dRk + off(R_L1 * 128), dBB, iKK64, 1u);
        umma_bf16(tmem + TM_G, dRk + off(R_L2 * 128), dBB, iKK64, 1u);
        umma_commit(smem_u32(&bars.d1_full));  // the reverse sweep can start
#ifdef NAJU_PROF
        {
          const long long t_a = clock64();
          mbar_wait(smem_u32(&bars.d1_full), par);
          atomicAdd(&g_profb[10], static_cast<unsigned long long>(clock64() - t_a));
        }
        const long long t_x = clock64();
#endif
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          // cross-channel: X[m, n'] += [al | wt]^T . [wt | h | lt]   (K = 16 channels per step);
          // these run on the tensor cores while the main warps do the sweep
          const uint64_t grp = dRm + off(2 * ks * SBO_R);
          umma_bf16(tmem + TM_X, grp + off(R_A1 * 128), grp + off(R_W1 * 128), iMM96, ks > 0);
          umma_bf16(tmem + TM_X, grp + off(R_A1 * 128), grp + off(R_W2 * 128), iMM96, 1u);
          umma_bf16(tmem + TM_X, grp + off(R_A2 * 128), grp + off(R_W1 * 128), iMM96, 1u);
        }
        umma_commit(smem_u32(&bars.d4_full));
#ifdef NAJU_PROF
        mbar_wait(smem_u32(&bars.d4_full), par);
        atomicAdd(&g_profb[11], static_cast<unsigned long long>(clock64() - t_x));
#endif
        // second round: the intra-chunk parts of dC and dB from the masked M2 the main warps wrote
        if (!mbar_wait(smem_u32(&bars.m2_full), par)) timeout();
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          // dCi[t,n] += sum_s M2[t,s] B[s,n]    (A = M2 rows, K = s)
          umma_bf16(tmem + TM_DCI, dMk + off((M_1 + 2 * ks) * 128), dBT + off(2 * ks * 128), iKK16, ks > 0);
          umma_bf16(tmem + TM_DCI, dMk + off((M_2 + 2 * ks) * 128), dBT + off(2 * ks * 128), iKK16, 1u);
          // dBi[64+s,n] += sum_t M2[t,s] C[t,n]   (A = M2 read MN-major, K = t)
          umma_bf16(tmem + TM_DBI, dMm + off(2 * ks * SBO_M + M_1 * 128), dCT + off(2 * ks * 128), iMK16, ks > 0);
          umma_bf16(tmem + TM_DBI, dMm + off(2 * ks * SBO_M + M_2 * 128), dCT + off(2 * ks * 128), iMK16, 1u);
        }
        umma_commit(smem_u32(&bars.d5_full));
      }
    }
  } else {
    // ===================================================================== main warps
    // Two threads per channel: warps 0-3 ("first half") own steps 0-31 of every chunk, warps 4-7
    // ("second half") steps 32-63; warps w and w+4 sit on the same TMEM lane quarter.  Neither half
    // waits for the other: the second half first runs a cheap product-only pass over steps 0-31 to
    // get R_32, and in the reverse sweep the first half first sums the r-increments of steps
    // 63-32 to get r_32.
    const int half = warp >> 2;
    const int cid = tid & (kDT - 1);  // channel within the tile
    const uint32_t trow = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    unsigned char* rows = smem + Smem::off_rows;
    unsigned char* my_row = rows + static_cast<uint32_t>(cid >> 3) * SBO_R + static_cast<uint32_t>(cid & 7) * 16;
    float lam[NS];  // adjoint entering the current chunk from the future (kept by both halves)
    float dDsum = 0.f;
    uint32_t slab = 0;
    PROFB_INIT;
    // dC / dB partial rows of the previous tile, written one tile late
    float UV[NS];
    int pend_t0 = 0, pend_len = 0, pend_b = 0, pend_dt = 0;
    uint32_t pend_par = 0;
    bool pending = false;
    auto flush_pending = [&]() {
      if (!pending) return;
      pending = false;
      if (!mbar_wait(smem_u32(&bars.d5_full), pend_par)) timeout();
      tc_fence_after();
      if (half == 0) {  // carry part (U, V) + intra-chunk part, one row per step of the chunk
        uint32_t x[16];
        tmem_ld16_async(trow + (cid < 64 ? TM_DCI : TM_DBI), x);
        tmem_ld_wait16(x);
        const int tt = cid & 63;
        if (tt < pend_len) {
          float* dst = (cid < 64 ? p.dCpart : p.dBpart) +
                       ((static_cast<int64_t>(pend_b) * p.T + pend_t0 + tt) * p.ndt + pend_dt) * NS;
#pragma unroll
          for (int q4 = 0; q4 < NS / 4; ++q4)
            reinterpret_cast<float4*>(dst)[q4] =
                make_float4(UV[4 * q4] + __uint_as_float(x[4 * q4]), UV[4 * q4 + 1] + __uint_as_float(x[4 * q4 + 1]),
                            UV[4 * q4 + 2] + __uint_as_float(x[4 * q4 + 2]), UV[4 * q4 + 3] + __uint_as_float(x[4 * q4 + 3]));
        }
      }
      tc_fence_before();
    };

    auto write_split_rows = [&](const float (&v)[NS], int c_hi, int c_lo) {
      uint32_t hi[8], lo[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) split_bf16x2(v[2 * k], v[2 * k + 1], hi[k], lo[k]);
      *reinterpret_cast<uint4*>(my_row + (c_hi + 0) * 128) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
      *reinterpret_cast<uint4*>(my_row + (c_hi + 1) * 128) = make_uint4(hi[4], hi[5], hi[6], hi[7]);
      *reinterpret_cast<uint4*>(my_row + (c_lo + 0) * 128) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
      *reinterpret_cast<uint4*>(my_row + (c_lo + 1) * 128) = make_uint4(lo[4], lo[5], lo[6], lo[7]);
    };

    float xe[NS], hv[NS];
    int it = 0;
    int x = x_first;
    do {
    // coordinates of the channel tile in hand
    const int xt = x, b = x / p.ndt, dt = x - b * p.ndt, d0 = dt * kDT, d = d0 + cid;
    const bool d_ok = d < p.D;
    const int cols = min(kDT, p.D - d0);
    const float Dv = d_ok ? __ldg(p.Dskip + d) : 0.f;
    // checkpointed states of a chunk: xe = state at its end (seed of the r recurrence, both
    // halves), hv = state entering it (first half only; h0 for the first chunk)
    auto fetch_states = [&](int c) {
      const int64_t tile = static_cast<int64_t>(c) * per_chunk + xt;
      const float4* src = reinterpret_cast<const float4*>(p.ckS + (tile * kDT + cid) * NS);
#pragma unroll
      for (int q4 = 0; q4 < NS / 4; ++q4) {
        const float4 v = __ldg(src + q4);
        xe[4 * q4] = v.x; xe[4 * q4 + 1] = v.y; xe[4 * q4 + 2] = v.z; xe[4 * q4 + 3] = v.w;
      }
      if (half == 0) {
        if (c > 0) {
          const float4* hs = reinterpret_cast<const float4*>(p.ckS + ((tile - per_chunk) * kDT + cid) * NS);
#pragma unroll
          for (int q4 = 0; q4 < NS / 4; ++q4) {
            const float4 v = __ldg(hs + q4);
            hv[4 * q4] = v.x; hv[4 * q4 + 1] = v.y; hv[4 * q4 + 2] = v.z; hv[4 * q4 + 3] = v.w;
          }
        } else {
#pragma unroll
          for (int n = 0; n < NS; ++n)
            hv[n] = (p.h0 != nullptr && d_ok && n < p.N) ? p.h0[(static_cast<int64_t>(b) * p.D + d) * p.N + n] : 0.f;
        }
      }
    };
#pragma unroll
    for (int n = 0; n < NS; ++n)
      lam[n] = (p.dhT != nullptr && d_ok && n < p.N) ? p.dhT[(static_cast<int64_t>(b) * p.D + d) * p.N + n] : 0.f;
    dDsum = 0.f;
    fetch_states(nchunks - 1);

    for (int ci = 0; ci < nchunks; ++ci, ++it) {
      const int c = nchunks - 1 - ci, t0 = c * Q, len = min(Q, p.T - t0);
      const uint32_t par = it & 1;
      // xe / hv (state at the chunk end / entering the chunk) were fetched during the previous
      // tile; the first half posts the h rows right away
      if (half == 0) write_split_rows(hv, R_H1, R_H2);
      PROFB_MARK(0);

      // ---------------- gates: operand rows [al | wt] and the coefficients the epilogue needs
      float R = 1.f;
#pragma unroll 1
      for (int k = 0; k < NSLAB; ++k) {
        const uint32_t sidx = slab + k, slot = sidx % RING, ph = (sidx / RING) & 1;
        const bool mine = (k >> 1) == half;
        // (every thread waits for the slab before releasing it, needed or not: an arrival must
        // not reach the empty barrier before its previous phase has completed)
        if (!mbar_wait(smem_u32(&bars.full[slot]), ph)) timeout();
        if (half == 0 && !mine) {  // first half: slabs 2,3 are not needed
          mbar_arrive(smem_u32(&bars.empty[slot]));
          continue;
        }
        const unsigned char* sl = smem + Smem::off_ring + slot * Smem::slab_bytes;
        const TA* s_u = reinterpret_cast<const TA*>(sl);
        const TG* s_fl = reinterpret_cast<const TG*>(sl + Smem::off_sfl);
        const TG* s_il = reinterpret_cast<const TG*>(sl + Smem::off_sil);
        const TA* s_dy = reinterpret_cast<const TA*>(sl + Smem::off_sdy);
        if (!mine) {
          // second half on slabs 0,1: retention products only, to enter step 32 with R_32
#pragma unroll
          for (int tl = 0; tl < SLAB; ++tl) {
            float a = fast_ex2(ld_as_f32(s_fl, tl * kDT + cid) * kNegLog2e);
            if (k * SLAB + tl >= len) a = 0.f;
            R *= 1.f + a;
          }
          mbar_arrive(smem_u32(&bars.empty[slot]));
          continue;
        }
        float Rprev = R;
#pragma unroll
        for (int j8 = 0; j8 < SLAB / 8; ++j8) {
          float wv[8], av[8];
          uint32_t cf[8], ci[8], cu[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int tl = 8 * j8 + j;
            const float flv = ld_as_f32(s_fl, tl * kDT + cid);
            const float ilv = fmaxf(ld_as_f32(s_il, tl * kDT + cid), -30.f);
            const float uv = ld_as_f32(s_u, tl * kDT + cid);
            const float dyv = ld_as_f32(s_dy, tl * kDT + cid);
            float a = fast_ex2(flv * kNegLog2e);
            const float bq = fast_ex2(ilv * kNegLog2e);
            if (k * SLAB + tl >= len) a = 0.f;       // ragged last chunk: neutral step (f = 1)
            const float opb = 1.f + bq;
            R *= 1.f + a;
            const float r = fast_rcp(R * opb);
            const float P = opb * r;                 // 1/R
            const float iR = R * r * R;              // i_t R_t
            wv[j] = uv * iR;
            av[j] = dyv * P;
            cf[j] = __float_as_uint(a * Rprev * P);  // 1 - f_t
            ci[j] = __float_as_uint(bq * (R * r));   // 1 - i_t
            cu[j] = __float_as_uint(iR);
            dDsum = fmaf(dyv, uv, dDsum);
            Rprev = R;
          }
          uint32_t h0, h1, h2, h3, l0, l1, l2, l3;
          const int ch = k * (SLAB / 8) + j8;
          split_bf16x2(av[0], av[1], h0, l0); split_bf16x2(av[2], av[3], h1, l1);
          split_bf16x2(av[4], av[5], h2, l2); split_bf16x2(av[6], av[7], h3, l3);
          *reinterpret_cast<uint4*>(my_row + (R_A1 + ch) * 128) = make_uint4(h0, h1, h2, h3);
          *reinterpret_cast<uint4*>(my_row + (R_A2 + ch) * 128) = make_uint4(l0, l1, l2, l3);
          split_bf16x2(wv[0], wv[1], h0, l0); split_bf16x2(wv[2], wv[3], h1, l1);
          split_bf16x2(wv[4], wv[5], h2, l2); split_bf16x2(wv[6], wv[7], h3, l3);
          *reinterpret_cast<uint4*>(my_row + (R_W1 + ch) * 128) = make_uint4(h0, h1, h2, h3);
          *reinterpret_cast<uint4*>(my_row + (R_W2 + ch) * 128) = make_uint4(l0, l1, l2, l3);
#define NAJU_TST8(COL, V)                                                                                   \
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(trow + (COL) + 8 * ch), \
               "r"(V[0]), "r"(V[1]), "r"(V[2]), "r"(V[3]), "r"(V[4]), "r"(V[5]), "r"(V[6]), "r"(V[7])          \
               : "memory")
          NAJU_TST8(TM_CF, cf);
          NAJU_TST8(TM_CI, ci);
          NAJU_TST8(TM_CU, cu);
#undef NAJU_TST8
        }
        mbar_arrive(smem_u32(&bars.empty[slot]));
        fence_async_smem();
        mbar_arrive(smem_u32(&bars.part[k]));  // the time-contraction MMAs of this slab may go
      }
      slab += NSLAB;
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      PROFB_MARK(1);
      if (half == 1) {
        if (!(R < kRMax)) atomicOr(&p.hdr->status, NAJU_ST_DEEP_TILE);  // never expected here
        const float PQ = fast_rcp(R);
        s_PQ[cid] = PQ;
        float lt[NS];
#pragma unroll
        for (int n = 0; n < NS; ++n) lt[n] = PQ * lam[n];
        write_split_rows(lt, R_L1, R_L2);
      }
      if (tid == 0) tma_store_wait_read();  // the previous tile's output tiles have left the staging area
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(smem_u32(&bars.carry_full));
      flush_pending();  // previous tile's dC / dB rows, while this tile's MMAs run
      PROFB_MARK(2);

      // ---------------- epilogue
      if (!mbar_wait(smem_u32(&bars.d1_full), par)) timeout();
      tc_fence_after();
      PROFB_MARK(3);
      // adjoint leaving the chunk, and the seed of the r recurrence
      float rr = 0.f;
      {
        uint32_t dl[16];
        tmem_ld16_async(trow + TM_DL, dl);
        tmem_ld_wait16(dl);
        const float PQ = s_PQ[cid];
#pragma unroll
        for (int n = 0; n < NS; ++n) {
          rr = fmaf(lam[n], xe[n], rr);
          lam[n] = fmaf(PQ, lam[n], __uint_as_float(dl[n]));
        }
      }
      if (c > 0) fetch_states(c - 1);  // next tile's states: the loads fly during the sweep
      PROFB_MARK(5);

      // reverse-time sweep, 8 steps per round: everything it needs comes from TMEM and this
      // thread's own operand row
      unsigned char* out_u = smem + Smem::off_out;
      unsigned char* out_f = out_u + Q * kDT * 2;
      unsigned char* out_i = out_f + Q * kDT * 2;
      const TA* gdy = reinterpret_cast<const TA*>(p.dy) + (static_cast<int64_t>(b) * p.T + t0) * p.D + d;
      TG* gdfl = reinterpret_cast<TG*>(p.dfl) + (static_cast<int64_t>(b) * p.T + t0) * p.D + d;
      TG* gdil = reinterpret_cast<TG*>(p.dil) + (static_cast<int64_t>(b) * p.T + t0) * p.D + d;
#define NAJU_TLD8(COL, V, CH)                                                                                \
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"                       \
               : "=r"(V[0]), "=r"(V[1]), "=r"(V[2]), "=r"(V[3]), "=r"(V[4]), "=r"(V[5]), "=r"(V[6]), "=r"(V[7]) \
               : "r"(trow + (COL) + 8 * (CH))                                                                 \
               : "memory")
#define NAJU_TWAIT16(A, B)                                                                                   \
  asm volatile("tcgen05.wait::ld.sync.aligned;"                                                              \
               : "+r"(A[0]), "+r"(A[1]), "+r"(A[2]), "+r"(A[3]), "+r"(A[4]), "+r"(A[5]), "+r"(A[6]), "+r"(A[7]), \
                 "+r"(B[0]), "+r"(B[1]), "+r"(B[2]), "+r"(B[3]), "+r"(B[4]), "+r"(B[5]), "+r"(B[6]), "+r"(B[7])  \
               :                                                                                             \
               : "memory")
#define NAJU_TWAIT8(A)                                                                                       \
  asm volatile("tcgen05.wait::ld.sync.aligned;"                                                              \
               : "+r"(A[0]), "+r"(A[1]), "+r"(A[2]), "+r"(A[3]), "+r"(A[4]), "+r"(A[5]), "+r"(A[6]), "+r"(A[7]) \
               :                                                                                             \
               : "memory")
      // TMEM loads are software-pipelined in both loops: the next round's columns are in flight
      // while the current round is processed.
      if (half == 0) {
        // first half: r-increments of steps 63..32 only, to enter step 31 with r_32
        uint32_t yq[2][8], gq[2][8];
        NAJU_TLD8(TM_Y, yq[1], Q / 8 - 1);
        NAJU_TLD8(TM_G, gq[1], Q / 8 - 1);
        NAJU_TWAIT16(yq[1], gq[1]);
#pragma unroll
        for (int ch = Q / 8 - 1; ch >= Q / 16; --ch) {
          const int cur = ch & 1, nxt = cur ^ 1;
          if (ch > Q / 16) {
            NAJU_TLD8(TM_Y, yq[nxt], ch - 1);
            NAJU_TLD8(TM_G, gq[nxt], ch - 1);
          }
          const uint4 a1 = *reinterpret_cast<const uint4*>(my_row + (R_A1 + ch) * 128);
          const uint4 a2 = *reinterpret_cast<const uint4*>(my_row + (R_A2 + ch) * 128);
          const uint4 w1 = *reinterpret_cast<const uint4*>(my_row + (R_W1 + ch) * 128);
          const uint4 w2 = *reinterpret_cast<const uint4*>(my_row + (R_W2 + ch) * 128);
          const uint32_t a1w[4] = {a1.x, a1.y, a1.z, a1.w}, a2w[4] = {a2.x, a2.y, a2.z, a2.w};
          const uint32_t w1w[4] = {w1.x, w1.y, w1.z, w1.w}, w2w[4] = {w2.x, w2.y, w2.z, w2.w};
#pragma unroll
          for (int j = 7; j >= 0; --j) {
            const uint32_t pa1 = a1w[j >> 1], pa2 = a2w[j >> 1], pw1 = w1w[j >> 1], pw2 = w2w[j >> 1];
            const float al = (j & 1) ? bf16hi_f32(pa1) + bf16hi_f32(pa2) : bf16lo_f32(pa1) + bf16lo_f32(pa2);
            const float wt = (j & 1) ? bf16hi_f32(pw1) + bf16hi_f32(pw2) : bf16lo_f32(pw1) + bf16lo_f32(pw2);
            rr += fmaf(al, __uint_as_float(yq[cur][j]), -wt * __uint_as_float(gq[cur][j]));
          }
          if (ch > Q / 16) NAJU_TWAIT16(yq[nxt], gq[nxt]);
        }
      }
      {
        const int ch_hi = half ? Q / 8 - 1 : Q / 16 - 1;
        uint32_t tq[2][5][8];
#define NAJU_TLOAD_ROUND(BUF, CH)          \
  do {                                     \
    NAJU_TLD8(TM_Y, tq[BUF][0], CH);       \
    NAJU_TLD8(TM_G, tq[BUF][1], CH);       \
    NAJU_TLD8(TM_CF, tq[BUF][2], CH);      \
    NAJU_TLD8(TM_CI, tq[BUF][3], CH);      \
    NAJU_TLD8(TM_CU, tq[BUF][4], CH);      \
  } while (0)
#define NAJU_TWAIT_ROUND(BUF)                  \
  do {                                         \
    NAJU_TWAIT16(tq[BUF][0], tq[BUF][1]);      \
    NAJU_TWAIT16(tq[BUF][2], tq[BUF][3]);      \
    NAJU_TWAIT8(tq[BUF][4]);                   \
  } while (0)
        NAJU_TLOAD_ROUND(0, ch_hi);
        NAJU_TWAIT_ROUND(0);
#pragma unroll
        for (int rd = 0; rd < Q / 16; ++rd) {
          const int ch = ch_hi - rd;
          const int cur = rd & 1, nxt = cur ^ 1;
          if (rd + 1 < Q / 16) NAJU_TLOAD_ROUND(nxt, ch - 1);
          const uint32_t* y8 = tq[cur][0];
          const uint32_t* g8 = tq[cur][1];
          const uint32_t* f8 = tq[cur][2];
          const uint32_t* i8 = tq[cur][3];
          const uint32_t* u8 = tq[cur][4];
          const uint4 a1 = *reinterpret_cast<const uint4*>(my_row + (R_A1 + ch) * 128);
          const uint4 a2 = *reinterpret_cast<const uint4*>(my_row + (R_A2 + ch) * 128);
          const uint4 w1 = *reinterpret_cast<const uint4*>(my_row + (R_W1 + ch) * 128);
          const uint4 w2 = *reinterpret_cast<const uint4*>(my_row + (R_W2 + ch) * 128);
          const uint32_t a1w[4] = {a1.x, a1.y, a1.z, a1.w}, a2w[4] = {a2.x, a2.y, a2.z, a2.w};
          const uint32_t w1w[4] = {w1.x, w1.y, w1.z, w1.w}, w2w[4] = {w2.x, w2.y, w2.z, w2.w};
#pragma unroll
          for (int j = 7; j >= 0; --j) {
            const int t = 8 * ch + j;
            const uint32_t pa1 = a1w[j >> 1], pa2 = a2w[j >> 1], pw1 = w1w[j >> 1], pw2 = w2w[j >> 1];
            const float al = (j & 1) ? bf16hi_f32(pa1) + bf16hi_f32(pa2) : bf16lo_f32(pa1) + bf16lo_f32(pa2);
            const float wt = (j & 1) ? bf16hi_f32(pw1) + bf16hi_f32(pw2) : bf16lo_f32(pw1) + bf16lo_f32(pw2);
            const float yt = __uint_as_float(y8[j]), gt = __uint_as_float(g8[j]);
            rr += fmaf(al, yt, -wt * gt);
            const float dfl = __uint_as_float(f8[j]) * rr;
            float du = __uint_as_float(u8[j]) * gt;
            if (Dv != 0.f && t < len) du = fmaf(Dv, to_f32(gdy[static_cast<int64_t>(t) * p.D]), du);
            const float dil = wt * __uint_as_float(i8[j]) * gt;
            reinterpret_cast<TA*>(out_u)[t * kDT + cid] = from_f32<TA>(du);
            if constexpr (Smem::kStageGates) {
              reinterpret_cast<TG*>(out_f)[t * kDT + cid] = from_f32<TG>(dfl);
              reinterpret_cast<TG*>(out_i)[t * kDT + cid] = from_f32<TG>(dil);
            } else if (d_ok && t < len) {
              gdfl[static_cast<int64_t>(t) * p.D] = from_f32<TG>(dfl);
              gdil[static_cast<int64_t>(t) * p.D] = from_f32<TG>(dil);
            }
          }
          if (rd + 1 < Q / 16) NAJU_TWAIT_ROUND(nxt);
        }
#undef NAJU_TLOAD_ROUND
#undef NAJU_TWAIT_ROUND
      }
#undef NAJU_TLD8
#undef NAJU_TWAIT16
#undef NAJU_TWAIT8
      PROFB_MARK(6);
      fence_async_smem();
      tc_fence_before();
      bar_sync<1, NMAIN>();
      if (tid == 0) {
        // du, d f_logit, d i_logit tiles out by TMA (steps past T and channels past D are clipped), one
        // bulk group each; the M2 operand re-uses the du tile, so wait until the du group has been read
        tma_store_3d(&maps.du, d0, t0, b, smem_u32(out_u));
        tma_store_commit();
        if constexpr (Smem::kStageGates) {
          tma_store_3d(&maps.dfl, d0, t0, b, smem_u32(out_f));
          tma_store_commit();
          tma_store_3d(&maps.dil, d0, t0, b, smem_u32(out_i));
          tma_store_commit();
          tma_store_wait_read_but<2>();
        } else {
          tma_store_wait_read();
        }
      }
      bar_sync<1, NMAIN>();  // the du tile has been read: the M2 operand may overwrite it
      PROFB_MARK(7);

      // ---------------- cross-channel block (its MMAs ran during the sweep): lanes t < 64 hold row t
      // of [M2 | U | .], lanes 64+s hold row s of [. | . | V]
      if (!mbar_wait(smem_u32(&bars.d4_full), par)) timeout();
      tc_fence_after();
      {
        uint32_t x[16];
        if (cid < 64) {
          // masked M2 row t as a two-term bf16 operand; each half writes 32 of the 64 columns
#pragma unroll
          for (int q2 = 0; q2 < 2; ++q2) {
            const int s16 = 2 * half + q2;
            tmem_ld16_async(trow + TM_X + 16 * s16, x);
            tmem_ld_wait16(x);
            uint32_t hi[8], lo[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const int s = 16 * s16 + 2 * k;
              split_bf16x2(s <= cid ? __uint_as_float(x[2 * k]) : 0.f, s + 1 <= cid ? __uint_as_float(x[2 * k + 1]) : 0.f,
                           hi[k], lo[k]);
            }
            unsigned char* mrow = smem + Smem::off_M + static_cast<uint32_t>(cid >> 3) * SBO_M + static_cast<uint32_t>(cid & 7) * 16;
            *reinterpret_cast<uint4*>(mrow + (M_1 + 2 * s16) * 128) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
            *reinterpret_cast<uint4*>(mrow + (M_1 + 2 * s16 + 1) * 128) = make_uint4(hi[4], hi[5], hi[6], hi[7]);
            *reinterpret_cast<uint4*>(mrow + (M_2 + 2 * s16) * 128) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            *reinterpret_cast<uint4*>(mrow + (M_2 + 2 * s16 + 1) * 128) = make_uint4(lo[4], lo[5], lo[6], lo[7]);
          }
        }
        if (half == 0) {
          tmem_ld16_async(trow + TM_X + (cid < 64 ? 64 : 80), x);  // U[t,:] or V[s,:]
          tmem_ld_wait16(x);
#pragma unroll
          for (int n = 0; n < NS; ++n) UV[n] = __uint_as_float(x[n]);
        }
      }
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(smem_u32(&bars.m2_full));
      PROFB_MARK(4);
      // The second MMA round (intra-chunk parts of dC / dB) is not waited for here: its result is
      // picked up while the next tile waits for its own first round.
      pend_t0 = t0;
      pend_len = len;
      pend_par = par;
      pend_b = b;
      pend_dt = dt;
      pending = true;
      tc_fence_before();
      // (the hazards of the next tile are all ordered by MMA barriers already; this barrier keeps
      // the eight warps in step, which measured 7 % faster than letting them drift)
      bar_sync<1, NMAIN>();
      PROFB_MARK(8);
    }
    // channel tile done: D_skip partials (one row per half and batch row), gradient of h0
    p.dDpart[(static_cast<int64_t>(half) * p.B + b) * (p.ndt * kDT) + d0 + cid] = dDsum;
    if (half == 0 && p.dh0 != nullptr && d_ok) {
      float* o = p.dh0 + (static_cast<int64_t>(b) * p.D + d) * p.N;
#pragma unroll
      for (int n = 0; n < NS; ++n)
        if (n < p.N) o[n] = lam[n];
    }
    x += x_step;
    } while (MULTI && x < per_chunk);
    flush_pending();
    if (tid == 0) tma_store_wait_all();
  }
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}

}  // namespace tcb

#ifdef NAJU_PROF
}  // namespace naju
extern "C" int naju_b200_debug_prof_bwd(unsigned long long* out16, int reset) {
  if (reset) {
    unsigned long long z[16] = {};
    return static_cast<int>(cudaMemcpyToSymbol(naju::tcb::g_profb, z, sizeof(z)));
  }
  return static_cast<int>(cudaMemcpyFromSymbol(out16, naju::tcb::g_profb, 16 * sizeof(unsigned long long)));
}
namespace naju {
#endif

// ------------------------------------------------------------------------------ host side
// Launches the tensor-core backward for this problem if it can take it; returns -1000 if not.
// The kernel itself stands down unless *fwd_form says the forward ran chunked without deep tiles.
namespace {
template <typename TA, typename TG>
int launch_bwd_tc_t(const BwdParams& p, const tcb::Maps& maps, const int* fwd_form, int64_t ctiles, cudaStream_t st) {
  constexpr size_t smem = tcb::SmemT<TG>::total;
  const bool multi = ctiles > tmah::sm_count();
  auto kern = multi ? tcb::bwd_tc_kernel<TA, TG, true> : tcb::bwd_tc_kernel<TA, TG, false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return static_cast<int>(e);
  const int64_t grid = std::min<int64_t>(ctiles, tmah::sm_count());
  kern<<<static_cast<unsigned>(grid), tcb::NTHREADS, smem, st>>>(p, maps, fwd_form);
  return static_cast<int>(cudaGetLastError());
}
}  // namespace

int launch_bwd_tc(const BwdParams& p, const Geometry& g, int act, int gate, int bc, const int* fwd_form,
                  void* stream) {
  if (!(g.N == tcb::NS && g.TC == tcb::Q && act == NAJU_BF16 && (gate == NAJU_BF16 || gate == NAJU_F32) &&
        bc == NAJU_BF16))
    return -1000;
  const int64_t ctiles = static_cast<int64_t>(g.B) * g.ndt;
  // One persistent CTA per SM walks whole channel tiles: with fewer than about a third of the SMs
  // busy the exact recurrent backward (which spreads over time as well) is the faster one.
  if (!(ctiles * 3 >= tmah::sm_count() && g.nchunks >= 4)) return -1000;
  tcb::Maps maps = {};
  const bool ok =
      tmah::make_map(&maps.u, p.u, act, g.B, g.T, g.D, p.u_sb, p.u_st, kDT, tcb::SLAB) &&
      tmah::make_map(&maps.fl, p.fl, gate, g.B, g.T, g.D, p.fl_sb, p.fl_st, kDT, tcb::SLAB) &&
      tmah::make_map(&maps.il, p.il, gate, g.B, g.T, g.D, p.il_sb, p.il_st, kDT, tcb::SLAB) &&
      tmah::make_map(&maps.dy, p.dy, act, g.B, g.T, g.D, static_cast<int64_t>(g.T) * g.D, g.D, kDT, tcb::SLAB) &&
      tmah::make_map(&maps.bm, p.Bm, bc, g.B, g.T, g.N, p.bm_sb, p.bm_st, tcb::NS, tcb::Q) &&
      tmah::make_map(&maps.cm, p.Cm, bc, g.B, g.T, g.N, p.cm_sb, p.cm_st, tcb::NS, tcb::Q) &&
      // outputs are dense [B, T, D]; one 64-step x 128-channel box per store (fp32 logit gradients
      // are written from registers, not by TMA)
      tmah::make_map(&maps.du, p.du, act, g.B, g.T, g.D, static_cast<int64_t>(g.T) * g.D, g.D, kDT, tcb::Q) &&
      (gate == NAJU_F32 ||
       (tmah::make_map(&maps.dfl, p.dfl, gate, g.B, g.T, g.D, static_cast<int64_t>(g.T) * g.D, g.D, kDT, tcb::Q) &&
        tmah::make_map(&maps.dil, p.dil, gate, g.B, g.T, g.D, static_cast<int64_t>(g.T) * g.D, g.D, kDT, tcb::Q)));
  if (!ok) return -1000;
  if (gate == NAJU_F32)
    return launch_bwd_tc_t<__nv_bfloat16, float>(p, maps, fwd_form, ctiles, static_cast<cudaStream_t>(stream));
  return launch_bwd_tc_t<__nv_bfloat16, __nv_bfloat16>(p, maps, fwd_form, ctiles, static_cast<cudaStream_t>(stream));
}

}  // namespace naju
