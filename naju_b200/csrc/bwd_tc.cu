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
// All contractions are tcgen05.mma (kind::f16, bf16 operands in two-term splits, fp32 accumulators
// in TMEM, M = 128).  Each channel owns one row [al | wt | h | lt] in shared memory; the same bytes
// serve as K-major operands for the per-channel GEMMs (contraction over time or state) and as
// MN-major operands for the cross-channel ones (contraction over the 128 channels); the G buffer
// serves K-major for Yt and MN-major (i.e. transposed) for gt, and the chunk's C and B rows serve
// K-major and MN-major alike, so nothing is ever transposed by hand.
//
// Twenty-four warps in five roles:
//   warps 0-15  main warps, four threads per channel: group g = warp / 4 owns steps [16g, 16g+16) of
//               every chunk, for the gates AND for the reverse sweep, so al_t and wt_t stay in its
//               registers in between.  Gates: the group multiplies up the retention of its own
//               steps, publishes the product and picks up the products of the groups before it
//               (no thread repeats another's steps); it writes its part of the channel's operand
//               row and the per-step coefficients (1-f_t), wt_t (1-i_t), i_t R_t (to TMEM).  Sweep,
//               once the first MMA round is complete: local suffix sums of al_t Yt_t - wt_t gt_t,
//               exchanged between the groups the same way, then d f_logit, du, d i_logit straight
//               to global memory (a warp's 32 channels are one contiguous piece per step).
//   warps 16-19 carry warps (thread = channel): adjoint carry lam, the checkpointed state entering
//               the chunk (h rows, posted as early as the previous tile allows), lt rows, the seed
//               of the r recurrence, dL -> lam; U / V of the cross-channel block and the chunk's
//               dC / dB partial rows after the second MMA round.
//   warps 20-21 operand builders: the chunk's C and B rows into operand layout, G = C B^T by one
//               tcgen05.mma of their own (M = time), read back row by row, masked, split in two
//               bf16 terms and written as the rows [C | g1 | g2]; double buffered, one tile ahead.
//               The same warps turn the cross-channel block's M2 into the masked two-term operand
//               of the second MMA round.
//   warp 22     TMA producer (input slabs of 16 steps: u, f_logit, i_logit, dy; raw B / C rows).
//   warp 23     MMA issuer (one thread; issuing from two warps was measured and is slower).
// Every wait is bounded.  Tiles with deep retention gates (prod f < 2^-80 in a chunk) cannot be
// factorised; the forward records whether it met one, and this kernel stands down in that case
// (the exact recurrent backward runs instead).
#include <algorithm>
#include <type_traits>

#include "common.cuh"
#include "params.h"
#include "tc_common.cuh"
#include "tma_host.h"

namespace naju {
namespace tcb {

using namespace tcx;

constexpr int Q = 64, NS = 16, SLAB = 16, NSLAB = Q / SLAB, NGRP = NSLAB, RING_MAX = 4;
constexpr int NMAIN = NGRP * 128, NCARRY = 128, NBUILD = 2;
constexpr int W_CARRY = NMAIN / 32, W_BUILD = W_CARRY + NCARRY / 32, W_PROD = W_BUILD + NBUILD, W_MMA = W_PROD + 1,
              NTHREADS = 32 * (W_MMA + 1);
static_assert(W_BUILD % 4 == 0, "builder warp k reads accumulator rows 32k .. 32k+31: its index must be k modulo 4");
// channel row (bf16, chunks of 8): [al1 8 | w1 8 | h1 2 | l1 2 | al2 8 | w2 8 | h2 2 | l2 2]
constexpr int R_A1 = 0, R_W1 = 8, R_H1 = 16, R_L1 = 18, R_A2 = 20, R_W2 = 28, R_H2 = 36, R_L2 = 38, R_CH = 40;
constexpr uint32_t SBO_R = R_CH * 128, ROWS_BYTES = 16 * SBO_R;  // 81920
// BG rows t: [C 2 | g1 8 | g2 8]
constexpr int BG_C = 0, BG_G1 = 2, BG_G2 = 10;
constexpr uint32_t SBO_BG = 18 * 128, BG_BYTES = 8 * SBO_BG;     // 18432
constexpr uint32_t SBO_BB = 2 * 128, BB_BYTES = 8 * SBO_BB;      // rows s: [B 2]        2048
// M2 operand rows t: [m1 8 | m2 8]; 64 real rows, addressed as 128 (the rest is never used)
constexpr int M_1 = 0, M_2 = 8;
constexpr uint32_t SBO_M = 16 * 128, M_BYTES = 8 * SBO_M;        // 16384
constexpr uint32_t BC_BYTES = Q * NS * 2;
// TMEM columns.  The intra-chunk parts of dC / dB (second MMA round) land in the first 32 columns of
// the cross-channel block, which has been read out by then.
// (dL sits directly before gt: one MMA with the B operand [C | g1] accumulates into both)
constexpr uint32_t TM_Y = 0, TM_DL = 64, TM_G = 80, TM_X = 144, TM_DCI = TM_X, TM_DBI = TM_X + 16, TM_CF = 240,
                   TM_CI = 304, TM_CU = 368, TM_GB = 432, TMEM_COLS = 512;
constexpr float kRMax = 1.0e24f;
constexpr float kNegLog2e = -1.4426950408889634f;
// Every wait parks the warp in mbarrier.try_wait (the hardware wakes it when the phase completes);
// sleeping 32-64 ns between polls instead, in any of the roles, was measured and is 4 % slower.

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

__device__ __forceinline__ uint32_t idesc_bf16(int N, uint32_t a_mn, uint32_t b_mn) {
  return umma_idesc(128, N, 1) | (a_mn << 15) | (b_mn << 16);
}

// packed fp32 pairs (one instruction for two lanes of arithmetic)
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 f2(uint32_t a, uint32_t b) { return make_float2(__uint_as_float(a), __uint_as_float(b)); }

// Two-term bf16 split of a pair: v ~= hi + lo, both truncations, so it costs integer and FMA-pipe
// operations only; residual <= 2^-16 relative.
__device__ __forceinline__ void split_pair(float2 v, uint32_t& hi, uint32_t& lo) {
  const uint32_t ua = __float_as_uint(v.x), ub = __float_as_uint(v.y);
  hi = __byte_perm(ua, ub, 0x7632);
  const float2 h = make_float2(__uint_as_float(ua & 0xFFFF0000u), __uint_as_float(ub & 0xFFFF0000u));
  const float2 l = fma2(h, make_float2(-1.f, -1.f), v);
  lo = __byte_perm(__float_as_uint(l.x), __float_as_uint(l.y), 0x7632);
}

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&v)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(v[0]), "r"(v[1]),
               "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]));
}

struct Maps {
  CUtensorMap u, fl, il, dy, bm, cm;
};

// TG = type of the logits and of their gradients.
template <typename TG>
struct SmemT {
  // Input slabs in flight.  A group waits for "its" slab by barrier parity, which is only sound if
  // the slot's previous use was filled before the group's own previous slab: RING >= NGRP.
  static constexpr int RING = 4;
  static_assert(RING >= NGRP, "");
  // Stages of the shared operand buffers: two with 16-bit logits (the builders run a tile ahead),
  // one with fp32 logits, whose input slabs need the room.
  static constexpr int NBG = sizeof(TG) == 2 ? 2 : 1;
  static constexpr uint32_t off_sfl = SLAB * kDT * 2;                       // slab: u | fl | il | dy
  static constexpr uint32_t off_sil = off_sfl + SLAB * kDT * sizeof(TG);
  static constexpr uint32_t off_sdy = off_sil + SLAB * kDT * sizeof(TG);
  static constexpr uint32_t slab_bytes = off_sdy + SLAB * kDT * 2;
  static constexpr uint32_t off_ring = 0;
  // The M2 operand is addressed as 128 rows (32 KB) although only 64 exist, and its MN-major view
  // starts eight chunks (1 KB) early: it sits between the ring and the channel rows, so both
  // overhangs are readable shared memory.  Likewise the builders' MMA reads the 64 C rows of a
  // stage as a 128-row operand: the operand buffers come before the channel rows too.
  static constexpr uint32_t off_BG = off_ring + RING * slab_bytes;   // [NBG]
  static constexpr uint32_t off_BB = off_BG + NBG * BG_BYTES;        // [NBG]
  static constexpr uint32_t off_bc = off_BB + NBG * BB_BYTES;        // [2 tiles][B raw | C raw]
  static constexpr uint32_t off_M = off_bc + 2 * 2 * BC_BYTES;
  static constexpr uint32_t off_rows = off_M + M_BYTES;
  static constexpr uint32_t total = off_rows + ROWS_BYTES;
  static_assert(off_M >= 8 * 128 && off_M + 16 * SBO_M <= total, "overhangs of the M2 operand stay inside shared memory");
  static_assert(off_BG + (NBG + 1) * BG_BYTES <= total, "the 128-row view of a stage's C rows stays inside shared memory");
};

struct Bars {
  unsigned long long full[RING_MAX], empty[RING_MAX];
  unsigned long long bc_full[2], bc_empty[2];
  unsigned long long lprod[NGRP];      // a group's retention product is published          (counts are in warps)
  unsigned long long ssum[NGRP];       // a group's sum of r-increments is published
  unsigned long long part[NSLAB];      // operand-row chunks of one 16-step slab written
  unsigned long long rq_ready;         // last group: the chunk's retention product is published
  unsigned long long h_full, lt_full;  // carry warps: h rows / lt rows written
  unsigned long long seed_ready[2];    // carry warps: seed of the r recurrence published
  unsigned long long ops_full[2];      // builders: C | g1 | g2 and B rows of a tile built
  unsigned long long g_full[2];        // the builders' own MMA is complete
  unsigned long long d1_full, d4_full; // MMA rounds complete: first (Yt, gt, dL), cross-channel
  unsigned long long d5_full[2];       // second round (and with it every read of the tile's BG / BB)
  unsigned long long m2_full;          // builders: M2 operand written; carry warps: U / V read
  unsigned long long x_free;           // carry warps: second-round results read
  unsigned long long acc_free;         // main + carry warps: Yt, gt, dL, coefficients read
};

template <typename TA, typename TG, bool UTM>
__global__ void __launch_bounds__(NTHREADS, 1)
bwd_tc_kernel(const BwdParams p, const __grid_constant__ Maps maps, const int* __restrict__ fwd_form) {
  using Smem = SmemT<TG>;
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ Bars bars;
  __shared__ unsigned int s_tmem;
  __shared__ float s_L[NGRP][kDT];   // retention product of a group's 16 steps (as 1 / prod f)
  __shared__ float s_S[NGRP][kDT];   // sum of the r-increments of a group's 16 steps
  __shared__ float s_Rend[kDT];      // 1 / (retention product of the whole chunk)
  __shared__ float s_seed[2][kDT];   // r at the chunk end: <lam, x_end>

  // stand down unless the forward ran in the chunked form and met no deep-gate tile
  if ((*fwd_form & 3) != 1) return;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t sbase = smem_u32(smem);
  // channel tiles (one batch row x 128 channels) are dealt round-robin over the grid; `it` counts
  // the (channel tile, chunk) pairs a CTA has seen and selects the barrier phases
  const int per_chunk = p.B * p.ndt;
  const int x_first = static_cast<int>(blockIdx.x), x_step = static_cast<int>(gridDim.x);
  const int nchunks = p.nchunks;
  const int ntotal = (x_first < per_chunk ? (per_chunk - x_first + x_step - 1) / x_step : 0) * nchunks;

  if (tid == 0) {
    if (blockIdx.x == 0) p.hdr->form = NAJU_FORM_TC_WALK;
    for (int i = 0; i < RING_MAX; ++i) {
      mbar_init(smem_u32(&bars.full[i]), 1);
      mbar_init(smem_u32(&bars.empty[i]), 4);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars.bc_full[i]), 1);
      mbar_init(smem_u32(&bars.bc_empty[i]), 1);
      mbar_init(smem_u32(&bars.seed_ready[i]), NCARRY / 32);
      mbar_init(smem_u32(&bars.ops_full[i]), NBUILD);
      mbar_init(smem_u32(&bars.g_full[i]), 1);
      mbar_init(smem_u32(&bars.d5_full[i]), 1);
    }
    for (int i = 0; i < NGRP; ++i) {
      mbar_init(smem_u32(&bars.lprod[i]), 4);
      mbar_init(smem_u32(&bars.ssum[i]), 4);
      mbar_init(smem_u32(&bars.part[i]), 4);
    }
    mbar_init(smem_u32(&bars.rq_ready), 4);
    mbar_init(smem_u32(&bars.h_full), NCARRY / 32);
    mbar_init(smem_u32(&bars.lt_full), NCARRY / 32);
    mbar_init(smem_u32(&bars.d1_full), 1);
    mbar_init(smem_u32(&bars.d4_full), 1);
    mbar_init(smem_u32(&bars.m2_full), NCARRY / 32 + NBUILD);
    mbar_init(smem_u32(&bars.x_free), NCARRY / 32);
    mbar_init(smem_u32(&bars.acc_free), NMAIN / 32 + NCARRY / 32);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(smem_u32(&s_tmem), TMEM_COLS);
  // zero the shared operand buffers and the M2 operand once: the upper triangles of g1/g2 and of
  // M2 are never written afterwards
  for (uint32_t i = tid * 16; i < Smem::NBG * (BG_BYTES + BB_BYTES); i += NTHREADS * 16)
    *reinterpret_cast<uint4*>(smem + Smem::off_BG + i) = make_uint4(0, 0, 0, 0);
  for (uint32_t i = tid * 16; i < M_BYTES; i += NTHREADS * 16)
    *reinterpret_cast<uint4*>(smem + Smem::off_M + i) = make_uint4(0, 0, 0, 0);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;
  auto timeout = [&]() { atomicOr(&p.hdr->status, NAJU_ST_MMA_TIMEOUT); };
  // u is time-contiguous: its slabs sit in shared memory as [channel][step], du goes out in the same
  // layout.  (A compile-time switch: as a run-time one it cost the usual layout registers and 18 %.)
  constexpr bool utm = UTM;

  if (warp == W_PROD) {
    // ===================================================================== TMA producer
    if (lane == 0) {
      uint32_t slab = 0;
      int it = 0;
      for (int x = x_first; x < per_chunk; x += x_step) {
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
            const uint32_t slot = slab % Smem::RING, ph = (slab / Smem::RING) & 1;
            if (slab >= Smem::RING && !mbar_wait(smem_u32(&bars.empty[slot]), ph ^ 1)) timeout();
            const uint32_t bar = smem_u32(&bars.full[slot]);
            const uint32_t dst = sbase + Smem::off_ring + slot * Smem::slab_bytes;
            mbar_arrive_expect_tx(bar, Smem::slab_bytes);
            // (a time-contiguous u is mapped (T, D, B): its slab lands as [channel][step])
            if (utm) tma_load_3d(dst, &maps.u, t0 + k * SLAB, d0, b, bar);
            else tma_load_3d(dst, &maps.u, d0, t0 + k * SLAB, b, bar);
            tma_load_3d(dst + Smem::off_sfl, &maps.fl, d0, t0 + k * SLAB, b, bar);
            tma_load_3d(dst + Smem::off_sil, &maps.il, d0, t0 + k * SLAB, b, bar);
            tma_load_3d(dst + Smem::off_sdy, &maps.dy, d0, t0 + k * SLAB, b, bar);
          }
        }
      }
    }
  } else if (warp >= W_BUILD && warp < W_BUILD + NBUILD) {
    // ===================================================================== operand builders
    // Trip k builds the shared operands of tile k (one tile ahead of the MMAs), then turns the
    // cross-channel block of tile k-1 into the masked M2 operand (rows 0-63 of that block sit on
    // these two warps' TMEM lanes).
    const int bw = warp - W_BUILD, t = bw * 32 + lane;   // the accumulator row (step) this thread reads back
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t idG = umma_idesc(128, Q, 1);
    // row t of a 64 x 64 accumulator block, masked to s <= t, in two bf16 terms -> chunks c_hi + c8 /
    // c_lo + c8 of row t of an operand buffer; chunks right of the diagonal stay zero (cleared once)
    auto tril_rows = [&](uint32_t tcol, unsigned char* row, int c_hi, int c_lo) {
      const int nch16 = 2 * (bw + 1);              // 16-column pieces up to this warp's last diagonal
#pragma unroll 1
      for (int c16 = 0; c16 < nch16; ++c16) {
        uint32_t x[16];
        tmem_ld16_async(tcol + 16 * c16, x);
        tmem_ld_wait16(x);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int c8 = 2 * c16 + h;
          if (c8 <= (t >> 3)) {
            uint32_t hi[4], lo[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const int s = 8 * c8 + 2 * k;
              split_pair(make_float2(s <= t ? __uint_as_float(x[8 * h + 2 * k]) : 0.f,
                                     s + 1 <= t ? __uint_as_float(x[8 * h + 2 * k + 1]) : 0.f), hi[k], lo[k]);
            }
            *reinterpret_cast<uint4*>(row + (c_hi + c8) * 128) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
            *reinterpret_cast<uint4*>(row + (c_lo + c8) * 128) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
          }
        }
      }
    };
    auto build = [&](int it) {
      {
        const int st = it % Smem::NBG, rb = it & 1;
        const uint32_t par = (it / Smem::NBG) & 1;
        if (!mbar_wait(smem_u32(&bars.bc_full[rb]), (it >> 1) & 1)) timeout();
        // stage st: every MMA of the tile NBG back that reads BG / BB (or the M2 operand) is complete
        if (it >= Smem::NBG && !mbar_wait(smem_u32(&bars.d5_full[st]), par ^ 1)) timeout();
        unsigned char* s_BG = smem + Smem::off_BG + st * BG_BYTES;
        unsigned char* s_BB = smem + Smem::off_BB + st * BB_BYTES;
        const __nv_bfloat16* Braw = reinterpret_cast<const __nv_bfloat16*>(smem + Smem::off_bc + rb * 2 * BC_BYTES);
        const __nv_bfloat16* Craw = Braw + Q * NS;
        // the chunk's C and B rows in operand layout: 32 bytes per row, two 16-byte pieces
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          *reinterpret_cast<uint4*>(s_BG + op_off16(t, BG_C * 8 + half * 8, SBO_BG)) =
              *reinterpret_cast<const uint4*>(Craw + t * NS + half * 8);
          *reinterpret_cast<uint4*>(s_BB + op_off16(t, half * 8, SBO_BB)) =
              *reinterpret_cast<const uint4*>(Braw + t * NS + half * 8);
        }
        fence_async_smem();
        tc_fence_before();
        bar_sync<3, 32 * NBUILD>();                  // both warps: rows written, last tile's G read
        tc_fence_after();
        if (bw == 0 && lane == 0) {
          mbar_arrive(smem_u32(&bars.bc_empty[rb]));  // the raw rows have been read
          // G[t, s] = <C_t, B_s>: M = 128 rows of which the 64 steps are real (the rest of the A
          // operand is whatever follows the C rows in shared memory; those accumulator rows are
          // never read), N = 64, K = 16 states
          umma_bf16(tmem + TM_GB, umma_desc(sbase + Smem::off_BG + st * BG_BYTES + BG_C * 128, 128, SBO_BG),
                    umma_desc(sbase + Smem::off_BB + st * BB_BYTES, 128, SBO_BB), idG, 0u);
          umma_commit(smem_u32(&bars.g_full[st]));
        }
        if (!mbar_wait(smem_u32(&bars.g_full[st]), par)) timeout();
        tc_fence_after();
        tril_rows(tmem + TM_GB + lane_off, s_BG + static_cast<uint32_t>(t >> 3) * SBO_BG + static_cast<uint32_t>(t & 7) * 16,
                  BG_G1, BG_G2);
        fence_async_smem();
        tc_fence_before();
        mbar_arrive_warp(smem_u32(&bars.ops_full[st]));
      }
    };
    auto m2_operand = [&](int it) {   // (it = the tile after the one whose block is read)
      {
        // the previous tile's cross-channel block is complete: tril(M2) as a two-term operand
        // (its last reader, that tile's predecessor's second round, was waited for above)
        if (!mbar_wait(smem_u32(&bars.d4_full), (it - 1) & 1)) timeout();
        tc_fence_after();
        tril_rows(tmem + TM_X + lane_off, smem + Smem::off_M + static_cast<uint32_t>(t >> 3) * SBO_M + static_cast<uint32_t>(t & 7) * 16,
                  M_1, M_2);
        fence_async_smem();
        tc_fence_before();
        mbar_arrive_warp(smem_u32(&bars.m2_full));
      }
    };
    // With two operand stages the build of tile k runs a tile ahead and comes first; with one stage
    // it has to wait for tile k-1's second MMA round, which needs that tile's M2 operand first.
    for (int it = 0; it <= ntotal; ++it) {
      if constexpr (Smem::NBG == 1) {
        if (it >= 1) m2_operand(it);
        if (it < ntotal) build(it);
      } else {
        if (it < ntotal) build(it);
        if (it >= 1) m2_operand(it);
      }
    }
  } else if (warp == W_MMA) {
    // ===================================================================== MMA issuer
    if (lane == 0) {
      const uint32_t aR = sbase + Smem::off_rows, aM = sbase + Smem::off_M;
      const uint32_t iKK64 = idesc_bf16(64, 0, 0), iKM64 = idesc_bf16(64, 0, 1), iKM80 = idesc_bf16(80, 0, 1),
                     iKM16 = idesc_bf16(16, 0, 1);
      const uint32_t iMM96 = idesc_bf16(96, 1, 1), iMM16 = idesc_bf16(16, 1, 1);
      // Every operand address is fixed, so the descriptors are built once; a descriptor for another
      // chunk / row group is the base plus (byte offset >> 4) in its address field.  K-major:
      // LBO = bytes between 16-byte K chunks, SBO = bytes between 8-row groups.  MN-major: LBO =
      // bytes between groups of 8 along K, SBO = bytes between 8-element chunks along M / N.
      const uint64_t dRk = umma_desc(aR, 128, SBO_R), dRm = umma_desc(aR, SBO_R, 128);     // channel rows
      // M2 operand: K-major as is; MN-major starting eight chunks early, so that column s lands in
      // accumulator row 64+s (the lane of the thread that holds V[s,:]); rows 0-63 are never read
      const uint64_t dMk = umma_desc(aM, 128, SBO_M), dMm = umma_desc(aM - 8 * 128, SBO_M, 128);
      auto off = [](uint32_t bytes) { return static_cast<uint64_t>(bytes >> 4); };
      // One tile's MMAs as straight-line code: the operand stage is a compile-time constant and
      // every slab loop is unrolled.  (Measured: the same MMAs issued from loops with a run-time
      // trip count or slab index take the kernel 10-15 % longer; an MMA of these shapes occupies
      // the tensor pipe for about fifty cycles whatever its N, so their number is what counts --
      // which is why dL rides along with gt in one instruction.)
      auto tile = [&](auto stc, int it) {
        constexpr uint32_t st = decltype(stc)::value;
        const uint32_t par = it & 1, par2 = (it / Smem::NBG) & 1;
        const uint32_t aBG = sbase + Smem::off_BG + st * BG_BYTES, aBB = sbase + Smem::off_BB + st * BB_BYTES;
        const uint64_t dGk = umma_desc(aBG, 128, SBO_BG), dGm = umma_desc(aBG, SBO_BG, 128);  // C | g1 | g2
        const uint64_t dCm = umma_desc(aBG + BG_C * 128, SBO_BG, 128);                        // C (| g1) read MN-major
        const uint64_t dBk = umma_desc(aBB, 128, SBO_BB), dBm = umma_desc(aBB, SBO_BB, 128);  // B rows
        if (!mbar_wait(smem_u32(&bars.ops_full[st]), par2)) timeout();
        // the accumulators and coefficients of the previous tile have been read
        if (it >= 1 && !mbar_wait(smem_u32(&bars.acc_free), par ^ 1)) timeout();
        // (and its second-round results, which sit in the columns of the cross-channel block: polled
        // here, long after they were read, rather than between the first round and that block)
        if (it >= 1 && !mbar_wait(smem_u32(&bars.x_free), par ^ 1)) timeout();
        // Yt = (h1 + h2).C   (K = n): the h rows are posted ahead of the tile
        if (!mbar_wait(smem_u32(&bars.h_full), par)) timeout();
        tc_fence_after();
        umma_bf16(tmem + TM_Y, dRk + off(R_H1 * 128), dGk + off(BG_C * 128), iKK64, 0u);
        umma_bf16(tmem + TM_Y, dRk + off(R_H2 * 128), dGk + off(BG_C * 128), iKK64, 1u);
        // the MMAs that contract over time need only the row chunks of their slab
#pragma unroll
        for (int ks = 0; ks < NSLAB; ++ks) {
          if (!mbar_wait(smem_u32(&bars.part[ks]), par)) timeout();
          tc_fence_after();
          // Yt += w1.g1 + w1.g2 + w2.g1   (K = s)
          const uint64_t g1 = dGk + off((BG_G1 + 2 * ks) * 128), g2 = dGk + off((BG_G2 + 2 * ks) * 128);
          umma_bf16(tmem + TM_Y, dRk + off((R_W1 + 2 * ks) * 128), g1, iKK64, 1u);
          umma_bf16(tmem + TM_Y, dRk + off((R_W1 + 2 * ks) * 128), g2, iKK64, 1u);
          umma_bf16(tmem + TM_Y, dRk + off((R_W2 + 2 * ks) * 128), g1, iKK64, 1u);
          // [dL | gt] += al1.[C | g1]^T + al2.[C | g1]^T,  gt += al1.g2^T   (K = t: the [C | g1 | g2]
          // buffer read MN-major; C and g1 are neighbours, so one MMA feeds both accumulators)
          const uint64_t cg1 = dCm + off(2 * ks * SBO_BG), g2t = dGm + off(2 * ks * SBO_BG + BG_G2 * 128);
          umma_bf16(tmem + TM_DL, dRk + off((R_A1 + 2 * ks) * 128), cg1, iKM80, ks > 0);
          umma_bf16(tmem + TM_G, dRk + off((R_A1 + 2 * ks) * 128), g2t, iKM64, 1u);
          umma_bf16(tmem + TM_DL, dRk + off((R_A2 + 2 * ks) * 128), cg1, iKM80, 1u);
        }
        // gt += (l1 + l2).B   (K = n): the only MMAs that need the whole chunk's retention product
        if (!mbar_wait(smem_u32(&bars.lt_full), par)) timeout();
        tc_fence_after();
        umma_bf16(tmem + TM_G, dRk + off(R_L1 * 128), dBk, iKK64, 1u);
        umma_bf16(tmem + TM_G, dRk + off(R_L2 * 128), dBk, iKK64, 1u);
        umma_commit(smem_u32(&bars.d1_full));  // the reverse sweep can start
        // cross-channel: X[m, n'] += [al | wt]^T . [wt | h | lt]   (K = 16 channels per step); these run
        // on the tensor cores while the main warps do the sweep
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t grp = dRm + off(2 * ks * SBO_R);
          umma_bf16(tmem + TM_X, grp + off(R_A1 * 128), grp + off(R_W1 * 128), iMM96, ks > 0);
          umma_bf16(tmem + TM_X, grp + off(R_A1 * 128), grp + off(R_W2 * 128), iMM96, 1u);
          umma_bf16(tmem + TM_X, grp + off(R_A2 * 128), grp + off(R_W1 * 128), iMM96, 1u);
        }
        umma_commit(smem_u32(&bars.d4_full));
        // second round: the intra-chunk parts of dC and dB from the masked M2 the builders wrote
        // (m2_full also says the cross-channel block has been read out of these columns)
        if (!mbar_wait(smem_u32(&bars.m2_full), par)) timeout();
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          // dCi[t,n] += sum_s M2[t,s] B[s,n]    (A = M2 rows, K = s; the B rows read MN-major)
          umma_bf16(tmem + TM_DCI, dMk + off((M_1 + 2 * ks) * 128), dBm + off(2 * ks * SBO_BB), iKM16, ks > 0);
          umma_bf16(tmem + TM_DCI, dMk + off((M_2 + 2 * ks) * 128), dBm + off(2 * ks * SBO_BB), iKM16, 1u);
          // dBi[64+s,n] += sum_t M2[t,s] C[t,n]   (A = M2 read MN-major, K = t; the C rows read MN-major)
          umma_bf16(tmem + TM_DBI, dMm + off(2 * ks * SBO_M + M_1 * 128), dCm + off(2 * ks * SBO_BG), iMM16, ks > 0);
          umma_bf16(tmem + TM_DBI, dMm + off(2 * ks * SBO_M + M_2 * 128), dCm + off(2 * ks * SBO_BG), iMM16, 1u);
        }
        umma_commit(smem_u32(&bars.d5_full[st]));
      };
      if constexpr (Smem::NBG == 2) {
        for (int it = 0; it < ntotal; it += 2) {
          tile(std::integral_constant<uint32_t, 0>{}, it);
          if (it + 1 < ntotal) tile(std::integral_constant<uint32_t, 1>{}, it + 1);
        }
      } else {
        for (int it = 0; it < ntotal; ++it) tile(std::integral_constant<uint32_t, 0>{}, it);
      }
    }
  } else if (warp >= W_CARRY && warp < W_BUILD) {
    // ===================================================================== carry warps
    const int cid = tid - W_CARRY * 32;   // channel within the tile = accumulator row of the cross-channel block
    const uint32_t trow = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    unsigned char* rows = smem + Smem::off_rows;
    unsigned char* my_row = rows + static_cast<uint32_t>(cid >> 3) * SBO_R + static_cast<uint32_t>(cid & 7) * 16;
    auto write_split_rows = [&](const float (&v)[NS], int c_hi, int c_lo) {
      uint32_t hi[8], lo[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) split_pair(make_float2(v[2 * k], v[2 * k + 1]), hi[k], lo[k]);
      *reinterpret_cast<uint4*>(my_row + (c_hi + 0) * 128) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
      *reinterpret_cast<uint4*>(my_row + (c_hi + 1) * 128) = make_uint4(hi[4], hi[5], hi[6], hi[7]);
      *reinterpret_cast<uint4*>(my_row + (c_lo + 0) * 128) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
      *reinterpret_cast<uint4*>(my_row + (c_lo + 1) * 128) = make_uint4(lo[4], lo[5], lo[6], lo[7]);
    };
    float lam[NS];   // adjoint entering the current chunk from the future
    float hv[NS];    // state entering the NEXT tile to post (= state at the end of the chunk before it)
    float seed = 0.f;
    // coordinates of the tile in hand
    int x = x_first, ci = 0;
    int b = 0, dt = 0, d = 0;
    bool d_ok = false;
    // state at the end of chunk c of channel tile xx (checkpoint; h0 below chunk 0)
    auto fetch_state = [&](int xx, int c, float (&v)[NS]) {
      const int bb = xx / p.ndt, dd = (xx - bb * p.ndt) * kDT + cid;
      if (c >= 0) {
        const int64_t tile = static_cast<int64_t>(c) * per_chunk + xx;
        const float4* src = reinterpret_cast<const float4*>(p.ckS + (tile * kDT + cid) * NS);
#pragma unroll
        for (int q4 = 0; q4 < NS / 4; ++q4) {
          const float4 t4 = __ldg(src + q4);
          v[4 * q4] = t4.x; v[4 * q4 + 1] = t4.y; v[4 * q4 + 2] = t4.z; v[4 * q4 + 3] = t4.w;
        }
      } else {
#pragma unroll
        for (int n = 0; n < NS; ++n)
          v[n] = (p.h0 != nullptr && dd < p.D && n < p.N) ? p.h0[(static_cast<int64_t>(bb) * p.D + dd) * p.N + n] : 0.f;
      }
    };
    // adjoint, seed and entering state of the last chunk of channel tile xx
    auto open_channel_tile = [&](int xx) {
      const int bb = xx / p.ndt, dd = (xx - bb * p.ndt) * kDT + cid;
#pragma unroll
      for (int n = 0; n < NS; ++n)
        lam[n] = (p.dhT != nullptr && dd < p.D && n < p.N) ? p.dhT[(static_cast<int64_t>(bb) * p.D + dd) * p.N + n] : 0.f;
      float xe[NS];
      fetch_state(xx, nchunks - 1, xe);
      seed = 0.f;
#pragma unroll
      for (int n = 0; n < NS; ++n) seed = fmaf(lam[n], xe[n], seed);
      fetch_state(xx, nchunks - 2, hv);
    };
    // h rows and the seed of the r recurrence of tile `jt` (from hv / seed)
    auto post_tile = [&](int jt) {
      write_split_rows(hv, R_H1, R_H2);
      fence_async_smem();
      mbar_arrive_warp(smem_u32(&bars.h_full));
      s_seed[jt & 1][cid] = seed;
      mbar_arrive_warp(smem_u32(&bars.seed_ready[jt & 1]));
    };
    if (ntotal > 0) {
      open_channel_tile(x);
      post_tile(0);
    }
#pragma unroll 1
    for (int it = 0; it < ntotal; ++it) {
      if (ci == 0) {
        b = x / p.ndt;
        dt = x - b * p.ndt;
        d = dt * kDT + cid;
        d_ok = d < p.D;
      }
      const int c = nchunks - 1 - ci, t0 = c * Q, len = min(Q, p.T - t0);
      const uint32_t par = it & 1, st = it % Smem::NBG, par2 = (it / Smem::NBG) & 1;
      // ---- the chunk's retention product is known: lt rows
      if (!mbar_wait(smem_u32(&bars.rq_ready), par)) timeout();
      const float Rend = s_Rend[cid];
      if (!(Rend < kRMax)) atomicOr(&p.hdr->status, NAJU_ST_DEEP_TILE);  // never expected here
      const float PQ = __frcp_rn(Rend);
      {
        float lt[NS];
#pragma unroll
        for (int n = 0; n < NS; ++n) lt[n] = PQ * lam[n];
        write_split_rows(lt, R_L1, R_L2);
      }
      fence_async_smem();
      mbar_arrive_warp(smem_u32(&bars.lt_full));
      // ---- first round complete: adjoint leaving the chunk; what the next tile starts from
      if (!mbar_wait(smem_u32(&bars.d1_full), par)) timeout();
      tc_fence_after();
      {
        uint32_t dl[16];
        tmem_ld16_async(trow + TM_DL, dl);
        tmem_ld_wait16(dl);
#pragma unroll
        for (int n = 0; n < NS; ++n) lam[n] = fmaf(PQ, lam[n], __uint_as_float(dl[n]));
      }
      tc_fence_before();
      mbar_arrive_warp(smem_u32(&bars.acc_free));
      const bool more = it + 1 < ntotal;
      if (c > 0) {
        // next tile = the chunk before this one: its r recurrence ends at <lam, state entering this
        // chunk>; the state entering it is one checkpoint further down
        seed = 0.f;
#pragma unroll
        for (int n = 0; n < NS; ++n) seed = fmaf(lam[n], hv[n], seed);
        fetch_state(x, c - 2, hv);
      } else {
        // channel tile done: gradient of h0; next tile = last chunk of the next channel tile
        if (p.dh0 != nullptr && d_ok) {
          float* o = p.dh0 + (static_cast<int64_t>(b) * p.D + d) * p.N;
#pragma unroll
          for (int n = 0; n < NS; ++n)
            if (n < p.N) o[n] = lam[n];
        }
        if (more) open_channel_tile(x + x_step);
      }
      // ---- cross-channel block complete, and with it every MMA that reads the channel rows: the
      // next tile's h rows go in right away (its first MMAs wait for nothing else from here)
      if (!mbar_wait(smem_u32(&bars.d4_full), par)) timeout();
      tc_fence_after();
      if (more) post_tile(it + 1);
      float UV[NS];
      {
        uint32_t xr[16];
        tmem_ld16_async(trow + TM_X + (cid < 64 ? 64 : 80), xr);  // U[t,:] or V[s,:]
        tmem_ld_wait16(xr);
#pragma unroll
        for (int n = 0; n < NS; ++n) UV[n] = __uint_as_float(xr[n]);
      }
      tc_fence_before();
      mbar_arrive_warp(smem_u32(&bars.m2_full));
      // ---- second round complete: carry part (U, V) + intra-chunk part, one row per step of the chunk
      if (!mbar_wait(smem_u32(&bars.d5_full[st]), par2)) timeout();
      tc_fence_after();
      {
        uint32_t xr[16];
        tmem_ld16_async(trow + (cid < 64 ? TM_DCI : TM_DBI), xr);
        tmem_ld_wait16(xr);
        const int tt = cid & 63;
        if (tt < len) {
          float* dst = (cid < 64 ? p.dCpart : p.dBpart) + ((static_cast<int64_t>(b) * p.T + t0 + tt) * p.ndt + dt) * NS;
#pragma unroll
          for (int q4 = 0; q4 < NS / 4; ++q4)
            reinterpret_cast<float4*>(dst)[q4] =
                make_float4(UV[4 * q4] + __uint_as_float(xr[4 * q4]), UV[4 * q4 + 1] + __uint_as_float(xr[4 * q4 + 1]),
                            UV[4 * q4 + 2] + __uint_as_float(xr[4 * q4 + 2]), UV[4 * q4 + 3] + __uint_as_float(xr[4 * q4 + 3]));
        }
      }
      tc_fence_before();
      mbar_arrive_warp(smem_u32(&bars.x_free));
      if (++ci == nchunks) {
        ci = 0;
        x += x_step;
      }
    }
  } else {
    // ===================================================================== main warps
    const int grp = warp >> 2;                     // owns steps [16 grp, 16 grp + 16) of every chunk
    const int cid = (warp & 3) * 32 + lane;        // channel within the tile
    const uint32_t trow = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16) + SLAB * grp;
    unsigned char* my_row = smem + Smem::off_rows + static_cast<uint32_t>(cid >> 3) * SBO_R + static_cast<uint32_t>(cid & 7) * 16;
    const float2 kk = make_float2(kNegLog2e, kNegLog2e), one2 = make_float2(1.f, 1.f);
    float dDsum = 0.f;
    int it = 0;
    for (int x = x_first; x < per_chunk; x += x_step) {
      const int b = x / p.ndt, dt = x - b * p.ndt, d0 = dt * kDT, d = d0 + cid;
      const bool d_ok = d < p.D;
      const float Dv = d_ok ? __ldg(p.Dskip + d) : 0.f;
      dDsum = 0.f;
#pragma unroll 1
      for (int ci = 0; ci < nchunks; ++ci, ++it) {
        const int c = nchunks - 1 - ci, t0 = c * Q, len = min(Q, p.T - t0);
        const uint32_t par = it & 1;
        const int nvalid = len - SLAB * grp;       // real steps among this thread's 16
        // the channel rows are free once every MMA of the previous tile that reads them is complete
        if (it >= 1 && !mbar_wait(smem_u32(&bars.d4_full), par ^ 1)) timeout();
        const uint32_t sidx = static_cast<uint32_t>(it) * NSLAB + grp, slot = sidx % Smem::RING, ph = (sidx / Smem::RING) & 1;
        if (!mbar_wait(smem_u32(&bars.full[slot]), ph)) timeout();
        const unsigned char* sl = smem + Smem::off_ring + slot * Smem::slab_bytes;
        const TA* s_u = reinterpret_cast<const TA*>(sl) + cid;          // [step][channel]
        const TA* s_ut = reinterpret_cast<const TA*>(sl) + cid * SLAB;   // [channel][step] (time-contiguous u)
        const TG* s_fl = reinterpret_cast<const TG*>(sl + Smem::off_sfl) + cid;
        const TG* s_il = reinterpret_cast<const TG*>(sl + Smem::off_sil) + cid;
        const TA* s_dy = reinterpret_cast<const TA*>(sl + Smem::off_sdy) + cid;
        // ---------------- gates (1): retention of the own 16 steps, a_j = e^{-f_logit_j},
        // L_j = prod_{i<=j} (1 + a_i), as pairs.  Steps past the end of the sequence (last chunk
        // only; they arrive as zeros from TMA) are made neutral: f = 1.
        float2 av[SLAB / 2], L[SLAB / 2];
#pragma unroll
        for (int j2 = 0; j2 < SLAB / 2; ++j2) {
          const float2 fl2 = mul2(make_float2(ld_as_f32(s_fl, (2 * j2) * kDT), ld_as_f32(s_fl, (2 * j2 + 1) * kDT)), kk);
          av[j2] = make_float2(fast_ex2(fl2.x), fast_ex2(fl2.y));
        }
        if (nvalid < SLAB) {
#pragma unroll
          for (int j2 = 0; j2 < SLAB / 2; ++j2) {
            if (2 * j2 >= nvalid) av[j2].x = 0.f;
            if (2 * j2 + 1 >= nvalid) av[j2].y = 0.f;
          }
        }
        {
          float run = 1.f;
#pragma unroll
          for (int j2 = 0; j2 < SLAB / 2; ++j2) {
            const float2 qv = add2(av[j2], one2);
            L[j2] = mul2(make_float2(run, run), make_float2(qv.x, qv.x * qv.y));
            run = L[j2].y;
          }
        }
        s_L[grp][cid] = L[SLAB / 2 - 1].y;
        mbar_arrive_warp(smem_u32(&bars.lprod[grp]));
        // ---------------- gates (2): R_t = (products of the groups before) x L_j; operand row chunks
        // [al | wt] of the own slab, per-step coefficients to TMEM; al_t and wt_t stay in registers
        float Rstart = 1.f;
        for (int g2 = 0; g2 < grp; ++g2) {
          if (!mbar_wait(smem_u32(&bars.lprod[g2]), par)) timeout();
          Rstart *= s_L[g2][cid];
        }
        const float2 Rs2 = make_float2(Rstart, Rstart);
        float2 alr[SLAB / 2], wtr[SLAB / 2];
#pragma unroll
        for (int j8 = 0; j8 < SLAB / 8; ++j8) {
          uint32_t ah[4], al_[4], wh[4], wl[4], cf[8], ci[8], cu[8];
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const int j2 = 4 * j8 + jj;
            const float2 il2 = mul2(make_float2(fmaxf(ld_as_f32(s_il, (2 * j2) * kDT), -30.f),
                                                fmaxf(ld_as_f32(s_il, (2 * j2 + 1) * kDT), -30.f)), kk);
            const float2 bq = make_float2(fast_ex2(il2.x), fast_ex2(il2.y));
            const float2 opb = add2(bq, one2);                      // 1 / i_t
            const float2 u2 = utm ? ld_pair_as_f32(s_ut + 2 * j2)
                                  : make_float2(ld_as_f32(s_u, (2 * j2) * kDT), ld_as_f32(s_u, (2 * j2 + 1) * kDT));
            const float2 dy2 = make_float2(ld_as_f32(s_dy, (2 * j2) * kDT), ld_as_f32(s_dy, (2 * j2 + 1) * kDT));
            const float2 R = mul2(Rs2, L[j2]);
            const float2 Rprev = make_float2(j2 == 0 ? Rstart : Rstart * L[j2 == 0 ? 0 : j2 - 1].y, R.x);
            const float2 x2 = mul2(R, opb);
            const float2 r = make_float2(fast_rcp(x2.x), fast_rcp(x2.y));
            const float2 P = mul2(opb, r);                          // 1 / R_t
            const float2 ig = mul2(R, r);                           // i_t
            const float2 iR = mul2(ig, R);                          // i_t R_t
            const float2 w = mul2(u2, iR);
            const float2 al = mul2(dy2, P);
            wtr[j2] = w;
            alr[j2] = al;
            const float2 cf2 = mul2(mul2(av[j2], Rprev), P);        // 1 - f_t
            const float2 ci2 = mul2(w, mul2(bq, ig));               // wt_t (1 - i_t)
            cf[2 * jj] = __float_as_uint(cf2.x); cf[2 * jj + 1] = __float_as_uint(cf2.y);
            ci[2 * jj] = __float_as_uint(ci2.x); ci[2 * jj + 1] = __float_as_uint(ci2.y);
            cu[2 * jj] = __float_as_uint(iR.x);  cu[2 * jj + 1] = __float_as_uint(iR.y);
            dDsum = fmaf(dy2.x, u2.x, fmaf(dy2.y, u2.y, dDsum));
            split_pair(al, ah[jj], al_[jj]);
            split_pair(w, wh[jj], wl[jj]);
          }
          const int ch = 2 * grp + j8;
          *reinterpret_cast<uint4*>(my_row + (R_A1 + ch) * 128) = make_uint4(ah[0], ah[1], ah[2], ah[3]);
          *reinterpret_cast<uint4*>(my_row + (R_A2 + ch) * 128) = make_uint4(al_[0], al_[1], al_[2], al_[3]);
          *reinterpret_cast<uint4*>(my_row + (R_W1 + ch) * 128) = make_uint4(wh[0], wh[1], wh[2], wh[3]);
          *reinterpret_cast<uint4*>(my_row + (R_W2 + ch) * 128) = make_uint4(wl[0], wl[1], wl[2], wl[3]);
          tmem_st8(trow + TM_CF + 8 * j8, cf);
          tmem_st8(trow + TM_CI + 8 * j8, ci);
          tmem_st8(trow + TM_CU + 8 * j8, cu);
        }
        mbar_arrive_warp(smem_u32(&bars.empty[slot]));   // the slab has been read
        if (grp == NGRP - 1) {
          s_Rend[cid] = Rstart * L[SLAB / 2 - 1].y;      // the whole chunk's product, for the carry warps
          mbar_arrive_warp(smem_u32(&bars.rq_ready));
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        fence_async_smem();
        mbar_arrive_warp(smem_u32(&bars.part[grp]));     // the time-contraction MMAs of this slab may go

        // ---------------- sweep (1), once the first MMA round is complete: z_t = al_t Yt_t - wt_t gt_t
        // and its suffix sums over the own steps, S_t = sum_{s >= t, own} z_s
        if (!mbar_wait(smem_u32(&bars.d1_full), par)) timeout();
        tc_fence_after();
        float2 S[SLAB / 2];
        {
          float run = 0.f;
#pragma unroll
          for (int j8 = SLAB / 8 - 1; j8 >= 0; --j8) {
            uint32_t y8[8], g8[8];
            tmem_ld8_async(trow + TM_Y + 8 * j8, y8);
            tmem_ld8_async(trow + TM_G + 8 * j8, g8);
            tmem_ld_wait8(y8, g8);
#pragma unroll
            for (int jj = 3; jj >= 0; --jj) {
              const int j2 = 4 * j8 + jj;
              const float2 wg = mul2(wtr[j2], f2(g8[2 * jj], g8[2 * jj + 1]));
              const float2 z = fma2(alr[j2], f2(y8[2 * jj], y8[2 * jj + 1]), make_float2(-wg.x, -wg.y));
              const float s1 = run + z.y;
              run = s1 + z.x;
              S[j2] = make_float2(run, s1);
            }
          }
          s_S[grp][cid] = run;
        }
        mbar_arrive_warp(smem_u32(&bars.ssum[grp]));
        // ---------------- sweep (2): r_t = seed + (sums of the groups after) + S_t; the three gradients
        if (!mbar_wait(smem_u32(&bars.seed_ready[it & 1]), (it >> 1) & 1)) timeout();
        float rstart = s_seed[it & 1][cid];
        for (int g2 = NGRP - 1; g2 > grp; --g2) {
          if (!mbar_wait(smem_u32(&bars.ssum[g2]), par)) timeout();
          rstart += s_S[g2][cid];
        }
        const float2 rs2 = make_float2(rstart, rstart), Dv2 = make_float2(Dv, Dv);
        const int64_t row0 = (static_cast<int64_t>(b) * p.T + t0 + SLAB * grp) * p.D + d;
        // (du of a time-contiguous u goes out in u's layout: this thread's 16 steps are 32 adjacent
        // bytes of its channel's row)
        TA* gdu = utm ? reinterpret_cast<TA*>(p.du) + static_cast<int64_t>(b) * p.u_sb + static_cast<int64_t>(d) * p.u_sd +
                            t0 + SLAB * grp
                      : reinterpret_cast<TA*>(p.du) + row0;
        TG* gdfl = reinterpret_cast<TG*>(p.dfl) + row0;
        TG* gdil = reinterpret_cast<TG*>(p.dil) + row0;
        const TA* gdy = reinterpret_cast<const TA*>(p.dy) + row0;
#pragma unroll
        for (int j8 = SLAB / 8 - 1; j8 >= 0; --j8) {
          uint32_t g8[8], f8[8], i8[8], u8[8];
          tmem_ld8_async(trow + TM_G + 8 * j8, g8);
          tmem_ld8_async(trow + TM_CF + 8 * j8, f8);
          tmem_ld_wait8(g8, f8);
          tmem_ld8_async(trow + TM_CI + 8 * j8, i8);
          tmem_ld8_async(trow + TM_CU + 8 * j8, u8);
          tmem_ld_wait8(i8, u8);
          [[maybe_unused]] uint32_t dupk[4];
#pragma unroll
          for (int jj = 3; jj >= 0; --jj) {
            const int j2 = 4 * j8 + jj, j = 2 * j2;
            const float2 gt = f2(g8[2 * jj], g8[2 * jj + 1]);
            const float2 dfl = mul2(f2(f8[2 * jj], f8[2 * jj + 1]), add2(S[j2], rs2));
            float2 du = mul2(f2(u8[2 * jj], u8[2 * jj + 1]), gt);
            const float2 dil = mul2(f2(i8[2 * jj], i8[2 * jj + 1]), gt);
            const bool ok0 = d_ok && j < nvalid, ok1 = d_ok && j + 1 < nvalid;
            if (Dv != 0.f) {
              const float y0 = ok0 ? to_f32(gdy[static_cast<int64_t>(j) * p.D]) : 0.f;
              const float y1 = ok1 ? to_f32(gdy[static_cast<int64_t>(j + 1) * p.D]) : 0.f;
              du = fma2(Dv2, make_float2(y0, y1), du);
            }
            if constexpr (utm) dupk[jj] = pack_bf16x2(du.x, du.y);
            if (ok0) {
              if constexpr (!utm) gdu[static_cast<int64_t>(j) * p.D] = from_f32<TA>(du.x);
              gdfl[static_cast<int64_t>(j) * p.D] = from_f32<TG>(dfl.x);
              gdil[static_cast<int64_t>(j) * p.D] = from_f32<TG>(dil.x);
            }
            if (ok1) {
              if constexpr (!utm) gdu[static_cast<int64_t>(j + 1) * p.D] = from_f32<TA>(du.y);
              gdfl[static_cast<int64_t>(j + 1) * p.D] = from_f32<TG>(dfl.y);
              gdil[static_cast<int64_t>(j + 1) * p.D] = from_f32<TG>(dil.y);
            }
          }
          if constexpr (utm) if (d_ok) {
            // eight steps of this channel's du: one 16-byte store when all of them are real
            if (8 * j8 + 8 <= nvalid) {
              *reinterpret_cast<uint4*>(gdu + 8 * j8) = make_uint4(dupk[0], dupk[1], dupk[2], dupk[3]);
            } else {
#pragma unroll
              for (int e = 0; e < 8; ++e)
                if (8 * j8 + e < nvalid)
                  reinterpret_cast<unsigned short*>(gdu)[8 * j8 + e] =
                      static_cast<unsigned short>(e & 1 ? dupk[e >> 1] >> 16 : dupk[e >> 1] & 0xFFFFu);
            }
          }
        }
        tc_fence_before();
        mbar_arrive_warp(smem_u32(&bars.acc_free));      // Yt, gt and the coefficients have been read
      }
      // channel tile done: D_skip partials (one row per group and batch row)
      p.dDpart[(static_cast<int64_t>(grp) * p.B + b) * (p.ndt * kDT) + d0 + cid] = dDsum;
    }
  }
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}

}  // namespace tcb

// ------------------------------------------------------------------------------ host side
// Launches the tensor-core backward for this problem if it can take it; returns -1000 if not.
// The kernel itself stands down unless *fwd_form says the forward ran chunked without deep tiles.
namespace {
template <typename TA, typename TG, bool UTM>
int launch_bwd_tc_t(const BwdParams& p, const tcb::Maps& maps, const int* fwd_form, int64_t ctiles, cudaStream_t st) {
  constexpr size_t smem = tcb::SmemT<TG>::total;
  auto kern = tcb::bwd_tc_kernel<TA, TG, UTM>;
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
  // One persistent CTA per SM walks whole channel tiles: with fewer than about a quarter of the SMs
  // busy the exact recurrent backward (which spreads over time as well) is the faster one
  // (measured at D=2048, T=65536: 48 channel tiles 22 against 15 M tokens/s, 32 tiles even).
  if (!(ctiles * 4 >= tmah::sm_count() && g.nchunks >= 4)) return -1000;
  tcb::Maps maps = {};
  const bool ok =
      (p.u_sd > 1 ? tmah::make_map_tmajor(&maps.u, p.u, act, g.B, g.T, g.D, p.u_sb, p.u_sd, tcb::SLAB, kDT)
                  : tmah::make_map(&maps.u, p.u, act, g.B, g.T, g.D, p.u_sb, p.u_st, kDT, tcb::SLAB)) &&
      tmah::make_map(&maps.fl, p.fl, gate, g.B, g.T, g.D, p.fl_sb, p.fl_st, kDT, tcb::SLAB) &&
      tmah::make_map(&maps.il, p.il, gate, g.B, g.T, g.D, p.il_sb, p.il_st, kDT, tcb::SLAB) &&
      tmah::make_map(&maps.dy, p.dy, act, g.B, g.T, g.D, static_cast<int64_t>(g.T) * g.D, g.D, kDT, tcb::SLAB) &&
      tmah::make_map(&maps.bm, p.Bm, bc, g.B, g.T, g.N, p.bm_sb, p.bm_st, tcb::NS, tcb::Q) &&
      tmah::make_map(&maps.cm, p.Cm, bc, g.B, g.T, g.N, p.cm_sb, p.cm_st, tcb::NS, tcb::Q);
  if (!ok) return -1000;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (p.u_sd > 1)
    return gate == NAJU_F32 ? launch_bwd_tc_t<__nv_bfloat16, float, true>(p, maps, fwd_form, ctiles, st)
                            : launch_bwd_tc_t<__nv_bfloat16, __nv_bfloat16, true>(p, maps, fwd_form, ctiles, st);
  return gate == NAJU_F32 ? launch_bwd_tc_t<__nv_bfloat16, float, false>(p, maps, fwd_form, ctiles, st)
                          : launch_bwd_tc_t<__nv_bfloat16, __nv_bfloat16, false>(p, maps, fwd_form, ctiles, st);
}

}  // namespace naju
