// Forward gated scan, chunked (state-expansion) form: persistent, TMA-fed, warp-specialised,
// tcgen05/TMEM, four threads per channel.
//
// Math (per chunk of Q = 64 steps, channel d; P_t = prod_{r<=t} f_r, R_t = 1/P_t,
// wt_s = sigmoid(i_s) u_s R_s; recurrence of naju/scan.py:79-93, contraction of
// naju/chunk_triton.py:79-144):
//     y_t   = P_t [ <C_t, h> + sum_{s<=t} (C_t . B_s) wt_s ] + D_skip u_t
//     x_end = P_Q [ h + sum_s wt_s B_s ]
// For 128 channels at once these are GEMMs with M = channel, issued as tcgen05.mma
// (kind::f16, bf16 operands, fp32 accumulators in TMEM):
//     D2[128 x 16] = (w1 + w2) . B^T                         chunk-local state increment
//     D1[128 x 64] = w1.g1 + w1.g2 + w2.g1 + (h1 + h2).C     pre-scaled outputs
// where wt = w1 + w2, tril(C B^T) = g1 + g2, h = h1 + h2 are two-term bf16 splits (16 mantissa
// bits; the dropped w2.g2 term is 2^-16 relative), so the tensor-core path keeps ~1e-5 accuracy.
//
// One persistent CTA per SM walks channel tiles (one batch row x 128 channels) along time, so
// the carry never leaves the chip.  Twenty-five warps in six roles; operand rows, shared operands
// and TMEM accumulators are double buffered (two pipeline stages):
//   warps 0-15  main warps, four threads per channel: group g = warp / 4 owns steps [16g, 16g+16) of
//               every chunk.  Per tile a thread (1) multiplies up the retention of its own 16
//               steps and publishes the product, (2) finishes the PREVIOUS tile for the same
//               steps -- y_t = P_t D1[d][t] (+ D_skip u_t) from TMEM into the staging tile; P_t is
//               still in its registers, so it never travels -- and (3) picks up the products of
//               the groups before it, which gives R_t, and writes its part of the channel's
//               operand row (K-major, no swizzle).  No thread repeats another thread's work.
//   warps 16-19 carry warps (thread = channel): D2 -> next chunk's carry-in (registers), the
//               checkpoint, and the carry-in operand row, posted one tile ahead; deep-gate tiles.
//   warps 20-21 operand builders: the chunk's C and B rows into operand layout, G = C B^T by one
//               tcgen05.mma of their own (M = time), read back from TMEM row by row (lane = step t),
//               masked to s <= t, split in two bf16 terms and written as the rows [C | g1 | g2].
//   warp 22     TMA producer: u / f_logit / i_logit in 16-step slabs (one per group) through an
//               mbarrier ring, and the chunk's raw B and C rows.
//   warp 23     MMA issuer: one thread issues every tcgen05.mma, slab by slab as the groups
//               deliver, and every tcgen05.commit.
//   warp 24     store warp: hands a finished staging tile to a TMA store and releases the stage
//               when the store has read it, so no compute warp ever waits for a store.
// A tile whose retention product falls below 2^-80 in any channel (deep gates) cannot use the
// 1/P_t factorisation; the carry warps then run the exact recurrence for that tile straight from
// global memory, from the carry they hold.  Every wait is bounded.
#include <algorithm>
#include <type_traits>

#include "fwd_common.cuh"
#include "tc_common.cuh"
#include "tma_host.h"

namespace naju {
namespace tc3 {

using namespace tcx;

constexpr int Q = 64, NS = 16, SLAB = 16, NSLAB = Q / SLAB, NSTAGE = 2;
#ifndef NAJU_RING16
#define NAJU_RING16 7
#endif
constexpr int RING_MAX = 8;                 // input-slab ring: as deep as shared memory allows (see Smem)
constexpr int NGRP = NSLAB;                 // main-warp groups: one slab of every chunk each
constexpr int NBUILD = 2;                   // operand-builder warps sharing a tile's work
constexpr int NHALF = 128, NMAIN = NGRP * 128, NCARRY = 128;
// (builder warp k reads accumulator rows 32k .. 32k+31: its index must be k modulo 4)
constexpr int W_CARRY = NMAIN / 32, W_BUILD = W_CARRY + NCARRY / 32, W_PROD = W_BUILD + NBUILD,
              W_MMA = W_PROD + 1, W_STORE = W_MMA + 1, NTHREADS = 32 * (W_STORE + 1);
static_assert(W_BUILD % 4 == 0 && NBUILD == 2, "builder warps sit on TMEM lane quarters 0 and 1");
constexpr int AW_W1 = 0, AW_W2 = 8;
constexpr uint32_t SBO_AW = 16 * 128, AW_BYTES = 16 * SBO_AW;  // operand rows [w1 64 | w2 64], per stage
constexpr int AH_H1 = 0, AH_H2 = 2;
constexpr uint32_t SBO_AH = 4 * 128, AH_BYTES = 16 * SBO_AH;   // carry-in rows [h1 16 | h2 16]
constexpr int B1_C = 0, B1_G1 = 2, B1_G2 = 10;
constexpr uint32_t SBO_B1 = 18 * 128, B1_BYTES = 8 * SBO_B1;   // rows t: [C 16 | g1 64 | g2 64]
constexpr uint32_t SBO_BB = 2 * 128, BB_BYTES = 8 * SBO_BB;    // rows s: [B 16]; read K-major (G) and MN-major (D2)
constexpr uint32_t BC_BYTES = Q * NS * 2;
constexpr uint32_t TM_D1 = 0, TM_D2 = 64, TM_P = 96, TM_G = 160, TM_STAGE = 224, TMEM_COLS = 512;
constexpr float kRMax = 1.0e24f;  // ~2^80
constexpr float kNegLog2e = -1.4426950408889634f;
// Every wait parks the warp in mbarrier.try_wait (the hardware wakes it when the phase completes);
// sleeping between polls instead, for the roles with slack, was measured and is 1 % slower.

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

struct Maps {
  CUtensorMap u, fl, il, bm, cm, y;
};

template <typename TG>
struct Smem {
  static constexpr uint32_t slab_bytes = SLAB * kDT * (2 + 2 * sizeof(TG));  // u, f_logit, i_logit
  // Input slabs are requested as far ahead as the ring is deep, and a slab is on its way for a
  // microsecond or more: with 16-bit logits the ring holds 7 slabs (1.75 tiles), with fp32 logits
  // (larger slabs) 4.
  static constexpr int RING = sizeof(TG) == 2 ? NAJU_RING16 : 4;
#ifndef NAJU_NY16
#define NAJU_NY16 1
#endif
  static constexpr int NY = sizeof(TG) == 2 ? NAJU_NY16 : 1;   // output staging tiles
  static constexpr uint32_t off_ring = 0;
  static constexpr uint32_t off_Y = off_ring + RING * slab_bytes;    // [NY][Q][128]
  // The builders' MMA addresses the 64 C rows of a stage as a 128-row operand: the 18 KB after a
  // stage's B1 buffer must be readable shared memory, so the large operand-row buffers come last.
  static constexpr uint32_t off_B1 = off_Y + NY * Q * kDT * 2;       // [NSTAGE]
  static constexpr uint32_t off_BB = off_B1 + NSTAGE * B1_BYTES;     // [NSTAGE]
  static constexpr uint32_t off_bc = off_BB + NSTAGE * BB_BYTES;     // [2 tiles][B raw | C raw]
  static constexpr uint32_t off_AH = off_bc + 2 * 2 * BC_BYTES;
  static constexpr uint32_t off_AW = off_AH + AH_BYTES;              // [NSTAGE]
  static constexpr uint32_t total = off_AW + NSTAGE * AW_BYTES;
  static_assert(off_B1 + (NSTAGE + 1) * B1_BYTES <= total, "the 128-row view of a stage's C rows stays inside shared memory");
};

struct Bars {
  unsigned long long full[RING_MAX], empty[RING_MAX];   // input slabs (producer <-> the group that owns the slab)
  unsigned long long bc_full[2], bc_empty[2];   // raw B/C rows per tile parity
  unsigned long long lprod[NSTAGE][NGRP];       // a group's retention products are published
  unsigned long long part[NSTAGE][NSLAB];       // operand-row chunks of one slab written (128 threads)
  unsigned long long g_full[NSTAGE];            // the builders' own MMA (G = C B^T) is complete
  unsigned long long ops_full[NSTAGE];          // builder -> MMA issuer
  unsigned long long d2_full[NSTAGE];           // D2 and the time-contraction part of D1 complete
  unsigned long long h_ready;                   // carry warps -> MMA issuer (carry-in row written)
  unsigned long long d1_full[NSTAGE];           // D1 complete (and the stage's shared operands read)
  unsigned long long y_staged[NSTAGE];          // main warps: outputs staged, accumulators read -> store warp, MMA issuer
  unsigned long long acc_free[NSTAGE];          // carry warps: D2 and the tile's flags read -> MMA issuer, last group
  unsigned long long stage_free[NSTAGE];        // store warp: staging tile read by the store -> epilogue two tiles on
};

// packed fp32 pairs (one instruction for two lanes of arithmetic)
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }

// Two-term bf16 split of a pair: v ~= hi + lo, both truncations (see split_bf16x2); packed subtraction.
__device__ __forceinline__ void split_pair(float2 v, uint32_t& hi, uint32_t& lo) {
  const uint32_t ua = __float_as_uint(v.x), ub = __float_as_uint(v.y);
  hi = __byte_perm(ua, ub, 0x7632);
  const float2 h = make_float2(__uint_as_float(ua & 0xFFFF0000u), __uint_as_float(ub & 0xFFFF0000u));
  const float2 l = fma2(h, make_float2(-1.f, -1.f), v);
  lo = __byte_perm(__float_as_uint(l.x), __float_as_uint(l.y), 0x7632);
}

// Exact recurrence of one tile straight from global memory (deep-gate tiles only), run by the 128
// carry threads from the carry they hold: hw / Pw = state and cumulative decay entering the chunk,
// updated to the chunk-end values (which are also written as the checkpoint).
template <typename TA, typename TG>
__device__ __noinline__ void exact_tile_from_global(const FwdParams& p, const TileCoord& tc, int tid,
                                                    float (&hw)[NS], float& Pw) {
  const TA* gu = reinterpret_cast<const TA*>(p.u) + tc.b * p.u_sb + static_cast<int64_t>(tc.t0) * p.u_st + tc.d * p.u_sd;
  const TG* gf = reinterpret_cast<const TG*>(p.fl) + tc.b * p.fl_sb + static_cast<int64_t>(tc.t0) * p.fl_st + tc.d;
  const TG* gi = reinterpret_cast<const TG*>(p.il) + tc.b * p.il_sb + static_cast<int64_t>(tc.t0) * p.il_st + tc.d;
  const int64_t bbase = tc.b * p.bm_sb + static_cast<int64_t>(tc.t0) * p.bm_st;
  const int64_t cbase = tc.b * p.cm_sb + static_cast<int64_t>(tc.t0) * p.cm_st;
  const float Dv = tc.d_ok ? p.Dskip[tc.d] : 0.f;
  TA* gy = reinterpret_cast<TA*>(p.y) + (static_cast<int64_t>(tc.b) * p.T + tc.t0) * p.D + tc.d;
  float Pc = 1.f;
  for (int t = 0; t < tc.len; ++t) {
    float f = 1.f, w = 0.f, ut = 0.f;
    if (tc.d_ok) {
      ut = to_f32(gu[t * p.u_st]);
      f = sigmoid_f(to_f32(gf[t * p.fl_st]));
      w = sigmoid_f(to_f32(gi[t * p.il_st])) * ut;
    }
    Pc *= f;
    float acc = 0.f;
#pragma unroll
    for (int n = 0; n < NS; ++n) {
      const float bv = n < p.N ? load_dyn(p.Bm, p.bc_dtype, bbase + t * p.bm_st + n) : 0.f;
      const float cv = n < p.N ? load_dyn(p.Cm, p.bc_dtype, cbase + t * p.cm_st + n) : 0.f;
      hw[n] = fmaf(f, hw[n], w * bv);
      acc = fmaf(cv, hw[n], acc);
    }
    if (tc.d_ok) gy[static_cast<int64_t>(t) * p.D] = from_f32<TA>(fmaf(Dv, ut, acc));
  }
  const int64_t slot = tc.tile * kDT + tid;
  float4* dstS = reinterpret_cast<float4*>(p.ckS + slot * NS);
#pragma unroll
  for (int q = 0; q < NS / 4; ++q) dstS[q] = make_float4(hw[4 * q], hw[4 * q + 1], hw[4 * q + 2], hw[4 * q + 3]);
  Pw *= Pc;
  p.ckP[slot] = Pw;
  write_final<NS>(p, tc, hw, Pw);
}

// Channel tiles (one batch row x 128 channels) are dealt round-robin over the grid; a CTA walks
// each of its channel tiles along time, chunk by chunk.  `it` counts the (channel tile, chunk)
// pairs a CTA has seen and selects the pipeline stage and barrier phases.
template <typename TA, typename TG, bool UTM>
__global__ void __launch_bounds__(NTHREADS, 1)
fwd_tc3_kernel(const FwdParams p, const __grid_constant__ Maps maps) {
  using SM = Smem<TG>;
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ Bars bars;
  __shared__ int s_stage_deep[NSTAGE];
  __shared__ int s_store_deep[NSTAGE];       // the same flag, handed to the store warp with the staged tile
  __shared__ unsigned int s_tmem;
  __shared__ float s_L[NSTAGE][NGRP][kDT];   // retention product of a group's 16 steps (as 1/prod f)
  __shared__ float s_Rend[NSTAGE][kDT];      // 1 / (retention product of the whole chunk)

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t sbase = smem_u32(smem);
  const int nchunks = p.nchunks, ctiles = p.B * p.ndt;
  const int x_first = static_cast<int>(blockIdx.x), x_step = static_cast<int>(gridDim.x);
  // (channel tile, chunk) pairs this CTA walks
  const int ntotal = (x_first < ctiles ? (ctiles - x_first + x_step - 1) / x_step : 0) * nchunks;

  if (tid == 0) {
    for (int i = 0; i < RING_MAX; ++i) {
      mbar_init(smem_u32(&bars.full[i]), 1);
      mbar_init(smem_u32(&bars.empty[i]), NHALF / 32);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars.bc_full[i]), 1);
      mbar_init(smem_u32(&bars.bc_empty[i]), 1);
    }
    for (int i = 0; i < NSTAGE; ++i) {
      for (int k = 0; k < NSLAB; ++k) {
        mbar_init(smem_u32(&bars.part[i][k]), NHALF / 32);     // (arrival counts are in warps)
        mbar_init(smem_u32(&bars.lprod[i][k]), NHALF / 32);
      }
      mbar_init(smem_u32(&bars.ops_full[i]), NBUILD);
      mbar_init(smem_u32(&bars.g_full[i]), 1);
      mbar_init(smem_u32(&bars.d2_full[i]), 1);
      mbar_init(smem_u32(&bars.d1_full[i]), 1);
      mbar_init(smem_u32(&bars.y_staged[i]), NMAIN / 32);
      mbar_init(smem_u32(&bars.acc_free[i]), NCARRY / 32);
      mbar_init(smem_u32(&bars.stage_free[i]), 1);   // (indexed by staging tile)
    }
    mbar_init(smem_u32(&bars.h_ready), NCARRY / 32);
    mbar_init_fence();
    if (blockIdx.x == 0) {
      atomicOr(p.fwd_form, 1);  // tell the backward how the forward ran
      p.hdr->form = NAJU_FORM_TC_WALK;
    }
  }
  if (warp == 0) tmem_alloc(smem_u32(&s_tmem), TMEM_COLS);
  // the upper triangle of g1/g2 is never written again: clear the shared operands once
  for (uint32_t i = tid * 16; i < NSTAGE * (B1_BYTES + BB_BYTES); i += NTHREADS * 16)
    *reinterpret_cast<uint4*>(smem + SM::off_B1 + i) = make_uint4(0, 0, 0, 0);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;
  auto timeout = [&]() { atomicOr(&p.hdr->status, NAJU_ST_MMA_TIMEOUT); };
  // u is time-contiguous: its slabs sit in shared memory as [channel][step].  (A compile-time
  // switch: as a run-time one it cost the usual layout 5 %.)
  constexpr bool utm = UTM;

  if (warp == W_PROD) {
    // ===================================================================== TMA producer
    if (lane == 0) {
      uint32_t slab = 0;
      int it = 0;
      for (int x = x_first; x < ctiles; x += x_step) {
        const int b = x / p.ndt, d0 = (x - b * p.ndt) * kDT;
        for (int c = 0; c < nchunks; ++c, ++it) {
          const int t0 = c * Q;
          if (it >= 2 && !mbar_wait(smem_u32(&bars.bc_empty[it & 1]), ((it >> 1) & 1) ^ 1)) timeout();
          {
            const uint32_t bar = smem_u32(&bars.bc_full[it & 1]);
            const uint32_t dst = sbase + SM::off_bc + (it & 1) * 2 * BC_BYTES;
            mbar_arrive_expect_tx(bar, 2 * BC_BYTES);
            tma_load_3d(dst, &maps.bm, 0, t0, b, bar);
            tma_load_3d(dst + BC_BYTES, &maps.cm, 0, t0, b, bar);
          }
          for (int k = 0; k < NSLAB; ++k, ++slab) {
            const uint32_t slot = slab % SM::RING, ph = (slab / SM::RING) & 1;
            if (slab >= SM::RING && !mbar_wait(smem_u32(&bars.empty[slot]), ph ^ 1)) timeout();
            const uint32_t bar = smem_u32(&bars.full[slot]);
            const uint32_t dst = sbase + SM::off_ring + slot * SM::slab_bytes;
            mbar_arrive_expect_tx(bar, SM::slab_bytes);
            // (a time-contiguous u is mapped (T, D, B): its slab lands as [channel][step])
            if (utm) tma_load_3d(dst, &maps.u, t0 + k * SLAB, d0, b, bar);
            else tma_load_3d(dst, &maps.u, d0, t0 + k * SLAB, b, bar);
            tma_load_3d(dst + SLAB * kDT * 2, &maps.fl, d0, t0 + k * SLAB, b, bar);
            tma_load_3d(dst + SLAB * kDT * (2 + sizeof(TG)), &maps.il, d0, t0 + k * SLAB, b, bar);
          }
        }
      }
    }
  } else if (warp >= W_BUILD && warp < W_BUILD + NBUILD) {
    // ===================================================================== operand builders
    const int bw = warp - W_BUILD, blane = bw * 32 + lane;
    const int t = blane;                           // the accumulator row (step) this thread reads back
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t idG = umma_idesc(128, Q, 1);
    for (int it = 0; it < ntotal; ++it) {
      const int st = it & 1;
      const uint32_t par = (it >> 1) & 1;
      if (!mbar_wait(smem_u32(&bars.bc_full[st]), par)) timeout();
      // stage st: the MMAs of the tile two back must have read B1 / BB (its epilogue may still run)
      if (it >= NSTAGE && !mbar_wait(smem_u32(&bars.d1_full[st]), par ^ 1)) timeout();
      unsigned char* s_B1 = smem + SM::off_B1 + st * B1_BYTES;
      unsigned char* s_BB = smem + SM::off_BB + st * BB_BYTES;
      const __nv_bfloat16* Braw = reinterpret_cast<const __nv_bfloat16*>(smem + SM::off_bc + st * 2 * BC_BYTES);
      const __nv_bfloat16* Craw = Braw + Q * NS;
      // the chunk's C and B rows in operand layout: 32 bytes per row, two 16-byte pieces
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        *reinterpret_cast<uint4*>(s_B1 + op_off16(t, B1_C * 8 + half * 8, SBO_B1)) =
            *reinterpret_cast<const uint4*>(Craw + t * NS + half * 8);
        *reinterpret_cast<uint4*>(s_BB + op_off16(t, half * 8, SBO_BB)) =
            *reinterpret_cast<const uint4*>(Braw + t * NS + half * 8);
      }
      fence_async_smem();
      tc_fence_before();
      bar_sync<3, 32 * NBUILD>();                  // both warps: rows written, last tile's G read
      tc_fence_after();
      if (blane == 0) {
        mbar_arrive(smem_u32(&bars.bc_empty[st]));  // the raw rows have been read
        // G[t, s] = <C_t, B_s>: M = 128 rows of which the 64 steps are real (the rest of the A
        // operand is whatever follows the C rows in shared memory; those accumulator rows are
        // never read), N = 64, K = 16 states
        umma_bf16(tmem + st * TM_STAGE + TM_G, umma_desc(sbase + SM::off_B1 + st * B1_BYTES + B1_C * 128, 128, SBO_B1),
                  umma_desc(sbase + SM::off_BB + st * BB_BYTES, 128, SBO_BB), idG, 0u);
        umma_commit(smem_u32(&bars.g_full[st]));
      }
      if (!mbar_wait(smem_u32(&bars.g_full[st]), par)) timeout();
      tc_fence_after();
      // row t of tril(G) in two bf16 terms -> [g1 | g2] of row t; chunks right of the diagonal stay
      // zero (cleared once, never written)
      unsigned char* row = s_B1 + static_cast<uint32_t>(t >> 3) * SBO_B1 + static_cast<uint32_t>(t & 7) * 16;
      const uint32_t tG = tmem + st * TM_STAGE + TM_G + lane_off;
      const int nch16 = 2 * (bw + 1);              // 16-column pieces up to this warp's last diagonal
#pragma unroll 1
      for (int c16 = 0; c16 < nch16; ++c16) {
        uint32_t x[16];
        tmem_ld16_async(tG + 16 * c16, x);
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
            *reinterpret_cast<uint4*>(row + (B1_G1 + c8) * 128) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
            *reinterpret_cast<uint4*>(row + (B1_G2 + c8) * 128) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
          }
        }
      }
      fence_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars.ops_full[st]));
    }
  } else if (warp == W_MMA) {
    // ===================================================================== MMA issuer
    if (lane == 0) {
      const uint32_t id16 = umma_idesc(128, NS, 1), id64 = umma_idesc(128, Q, 1);
      // operand addresses are fixed: build the descriptors once, offset the address field per use
      const uint64_t dAW0 = umma_desc(sbase + SM::off_AW, 128, SBO_AW), dAH = umma_desc(sbase + SM::off_AH, 128, SBO_AH);
      const uint64_t dB10 = umma_desc(sbase + SM::off_B1, 128, SBO_B1);
      // the B rows read MN-major (N = state contiguous, K = step): LBO = bytes between 8-step groups,
      // SBO = bytes between 8-state chunks
      const uint64_t dBB0 = umma_desc(sbase + SM::off_BB, SBO_BB, 128);
      const uint32_t id16m = id16 | (1u << 16);
      auto off = [](uint32_t bytes) { return static_cast<uint64_t>(bytes >> 4); };
      for (int it = 0; it < ntotal; ++it) {
        const int st = it & 1;
        const uint32_t par = (it >> 1) & 1;
        const uint64_t dAW = dAW0 + off(st * AW_BYTES), dB1 = dB10 + off(st * B1_BYTES), dBB = dBB0 + off(st * BB_BYTES);
        const uint32_t tst = tmem + st * TM_STAGE;
        if (!mbar_wait(smem_u32(&bars.ops_full[st]), par)) timeout();
        // the stage's accumulators: every reader of the tile two back is done with them
        if (it >= NSTAGE && !mbar_wait(smem_u32(&bars.y_staged[st]), par ^ 1)) timeout();
        if (it >= NSTAGE && !mbar_wait(smem_u32(&bars.acc_free[st]), par ^ 1)) timeout();
#pragma unroll 1
        for (int ks = 0; ks < NSLAB; ++ks) {
          // the time contractions of slab ks run while the other groups are still on their slabs
          if (!mbar_wait(smem_u32(&bars.part[st][ks]), par)) timeout();
          tc_fence_after();
          const uint64_t w1 = dAW + off((AW_W1 + 2 * ks) * 128), w2 = dAW + off((AW_W2 + 2 * ks) * 128);
          umma_bf16(tst + TM_D2, w1, dBB + off(2 * ks * SBO_BB), id16m, ks > 0);   // D2 += (w1 + w2) . B^T
          umma_bf16(tst + TM_D2, w2, dBB + off(2 * ks * SBO_BB), id16m, 1u);
          umma_bf16(tst + TM_D1, w1, dB1 + off((B1_G1 + 2 * ks) * 128), id64, ks > 0);  // D1 += w1.g1 + w1.g2 + w2.g1
          umma_bf16(tst + TM_D1, w1, dB1 + off((B1_G2 + 2 * ks) * 128), id64, 1u);
          umma_bf16(tst + TM_D1, w2, dB1 + off((B1_G1 + 2 * ks) * 128), id64, 1u);
        }
        // all four slabs are in: D2 is complete when these MMAs are
        umma_commit(smem_u32(&bars.d2_full[st]));
        // (the accumulators of a deep-gate tile are junk and are simply never read; the carry-in MMAs
        // run for it all the same, which keeps the barrier phases aligned)
        if (!mbar_wait(smem_u32(&bars.h_ready), it & 1)) timeout();
        tc_fence_after();
        umma_bf16(tst + TM_D1, dAH + off(AH_H1 * 128), dB1 + off(B1_C * 128), id64, 1u);  // D1 += (h1 + h2) . C
        umma_bf16(tst + TM_D1, dAH + off(AH_H2 * 128), dB1 + off(B1_C * 128), id64, 1u);
        umma_commit(smem_u32(&bars.d1_full[st]));
      }
    }
  } else if (warp == W_STORE) {
    // ===================================================================== store warp
    if (lane == 0) {
      int it = 0;
      for (int x = x_first; x < ctiles; x += x_step) {
        const int b = x / p.ndt, d0 = (x - b * p.ndt) * kDT;
        for (int c = 0; c < nchunks; ++c, ++it) {
          const int st = it & 1;
          if (!mbar_wait(smem_u32(&bars.y_staged[st]), (it >> 1) & 1)) timeout();
          if (!s_store_deep[st]) {
            // the staged tile leaves by TMA (steps past T and channels past D are clipped); the stage
            // is released once the store has read it
            tma_store_3d(&maps.y, d0, c * Q, b, sbase + SM::off_Y + (it % SM::NY) * Q * kDT * 2);
            tma_store_commit();
            tma_store_wait_read();
          }
          mbar_arrive(smem_u32(&bars.stage_free[it % SM::NY]));
        }
      }
      tma_store_wait_all();
    }
  } else if (warp >= W_CARRY) {
    // ===================================================================== carry warps
    const int q = tid - W_CARRY * 32;     // channel within the tile
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    unsigned char* h_row = smem + SM::off_AH + static_cast<uint32_t>(q >> 3) * SBO_AH + static_cast<uint32_t>(q & 7) * 16;
    auto write_h_row = [&](const float (&hv)[NS]) {
      uint32_t hi[8], lo[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) split_pair(make_float2(hv[2 * k], hv[2 * k + 1]), hi[k], lo[k]);
      *reinterpret_cast<uint4*>(h_row + (AH_H1 + 0) * 128) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
      *reinterpret_cast<uint4*>(h_row + (AH_H1 + 1) * 128) = make_uint4(hi[4], hi[5], hi[6], hi[7]);
      *reinterpret_cast<uint4*>(h_row + (AH_H2 + 0) * 128) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
      *reinterpret_cast<uint4*>(h_row + (AH_H2 + 1) * 128) = make_uint4(lo[4], lo[5], lo[6], lo[7]);
      fence_async_smem();
      tc_fence_before();
      mbar_arrive_warp(smem_u32(&bars.h_ready));
    };
    // state / cumulative decay entering the current chunk
    float hc[NS];
    float Pc = 1.f;
    auto load_h0 = [&](int x) {  // carry-in of the first chunk of channel tile x
      const int b = x / p.ndt, d = (x - b * p.ndt) * kDT + q;
#pragma unroll
      for (int n = 0; n < NS; ++n)
        hc[n] = (p.h0 != nullptr && d < p.D && n < p.N) ? p.h0[(static_cast<int64_t>(b) * p.D + d) * p.N + n] : 0.f;
      Pc = 1.f;
    };
    // One carry-in row (one h_ready phase) is posted per tile, one tile ahead.
    if (x_first < ctiles) {
      load_h0(x_first);
      write_h_row(hc);
    }
    int it = 0;
    for (int x = x_first; x < ctiles; x += x_step) {
      TileCoord tcd;
      tcd.per_chunk = ctiles;
      tcd.rem = x;
      tcd.b = x / p.ndt;
      tcd.dt = x - tcd.b * p.ndt;
      tcd.d0 = tcd.dt * kDT;
      tcd.cols = min(kDT, p.D - tcd.d0);
      tcd.d = tcd.d0 + q;
      tcd.d_ok = tcd.d < p.D;
      for (int c = 0; c < nchunks; ++c, ++it) {
        const int st = it & 1;
        if (!mbar_wait(smem_u32(&bars.d2_full[st]), (it >> 1) & 1)) timeout();
        if (!mbar_wait(smem_u32(&bars.part[st][NGRP - 1]), (it >> 1) & 1)) timeout();  // (the writers of s_Rend arrived here)
        tcd.c = c;
        tcd.tile = static_cast<int64_t>(c) * ctiles + x;
        tcd.t0 = c * Q;
        tcd.len = min(Q, p.T - tcd.t0);
        // 1 / (the chunk's retention product), from the last group; a tile where it overflowed in any
        // channel (deep gates) cannot use the factorisation
        const float Rend = s_Rend[st][q];
        const bool deep = bar_or<2, NCARRY>(!(Rend < kRMax));
        if (q == 0) s_stage_deep[st] = deep ? 1 : 0;
        tc_fence_after();
        if (deep) {
          if (q == 0) atomicOr(p.fwd_form, 2);
          exact_tile_from_global<TA, TG>(p, tcd, q, hc, Pc);
        } else {
          // chunk aggregate from D2: chunk-end state = next carry-in = checkpoint
          uint32_t sr[16];
          tmem_ld16_async(tmem + st * TM_STAGE + lane_off + TM_D2, sr);
          tmem_ld_wait16(sr);
          const float P = __frcp_rn(Rend);
#pragma unroll
          for (int n = 0; n < NS; ++n) hc[n] = P * (hc[n] + __uint_as_float(sr[n]));
          const int64_t slot = tcd.tile * kDT + q;
          float4* dstS = reinterpret_cast<float4*>(p.ckS + slot * NS);
#pragma unroll
          for (int q4 = 0; q4 < NS / 4; ++q4)
            dstS[q4] = make_float4(hc[4 * q4], hc[4 * q4 + 1], hc[4 * q4 + 2], hc[4 * q4 + 3]);
          Pc *= P;
          p.ckP[slot] = Pc;
          write_final<NS>(p, tcd, hc, Pc);
        }
        // D2 and s_Rend have been read, the tile's deep flag is written: one arrival per warp
        tc_fence_before();
        mbar_arrive_warp(smem_u32(&bars.acc_free[st]));
        if (!mbar_wait(smem_u32(&bars.d1_full[st]), (it >> 1) & 1)) timeout();
        // the last MMA of this tile has read the carry-in row: post the next tile's row now
        if (c + 1 < nchunks) {
          write_h_row(hc);
        } else if (x + x_step < ctiles) {
          load_h0(x + x_step);
          write_h_row(hc);
        }
      }
    }
  } else {
    // ===================================================================== main warps
    const int grp = warp >> 2;                     // owns steps [16 grp, 16 grp + 16) of every chunk
    const int q = (warp & 3) * 32 + lane;          // channel within the tile
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const float2 kk = make_float2(kNegLog2e, kNegLog2e), one2 = make_float2(1.f, 1.f);
    // the tile whose epilogue is pending (it runs one tile late, after the next tile's operand rows)
    int e_b = 0, e_d0 = 0, e_t0 = 0, e_len = 0, e_it = -1;
    float e_Dv = 0.f;

    auto epilogue = [&]() {
      // y_t = P_t D1[d][t] + D_skip u_t for this thread's 16 steps of the pending tile, into the
      // stage's staging tile (step t -> 256 contiguous bytes); P_t comes back from TMEM
      const int st = e_it & 1;
      const uint32_t par = (e_it >> 1) & 1;
      if (!mbar_wait(smem_u32(&bars.acc_free[st]), par)) timeout();   // (the deep flag's writers arrived here)
      if (!mbar_wait(smem_u32(&bars.d1_full[st]), par)) timeout();
      // the staging tile was last used NY tiles back: that store must have read it
      const int ys = e_it % SM::NY;
      if (e_it >= SM::NY && !mbar_wait(smem_u32(&bars.stage_free[ys]), ((e_it / SM::NY) & 1) ^ 1)) timeout();
      tc_fence_after();
      const bool deep = s_stage_deep[st] != 0;
      if (tid == 0) s_store_deep[st] = deep ? 1 : 0;
      if (!deep) {
        uint32_t v[SLAB], pv[SLAB];
        const uint32_t tb = tmem + st * TM_STAGE + lane_off + SLAB * grp;
        tmem_ld16_async(tb + TM_D1, v);
        tmem_ld16_async(tb + TM_P, pv);
        unsigned char* dst = smem + SM::off_Y + ys * (Q * kDT * 2) + (SLAB * grp) * (kDT * 2) + q * 2;
        const TA* gu = reinterpret_cast<const TA*>(p.u) + e_b * p.u_sb + static_cast<int64_t>(e_t0 + SLAB * grp) * p.u_st +
                       static_cast<int64_t>(e_d0 + q) * p.u_sd;
        tmem_ld_wait16(v);
        tmem_ld_wait16(pv);
#pragma unroll
        for (int j2 = 0; j2 < SLAB / 2; ++j2) {
          float2 y = mul2(make_float2(__uint_as_float(pv[2 * j2]), __uint_as_float(pv[2 * j2 + 1])),
                          make_float2(__uint_as_float(v[2 * j2]), __uint_as_float(v[2 * j2 + 1])));
          if (e_Dv != 0.f) {  // (the mixer passes a zero D_skip: naju/mixer.py:120-124)
            const int t = SLAB * grp + 2 * j2;
            float u0 = 0.f, u1 = 0.f;
            if (t < e_len) u0 = to_f32(gu[static_cast<int64_t>(2 * j2) * p.u_st]);
            if (t + 1 < e_len) u1 = to_f32(gu[static_cast<int64_t>(2 * j2 + 1) * p.u_st]);
            y = fma2(make_float2(e_Dv, e_Dv), make_float2(u0, u1), y);
          }
          unsigned short o0, o1;
          if constexpr (std::is_same<TA, __nv_bfloat16>::value) {
            const uint32_t pk = pack_bf16x2(y.x, y.y);  // one conversion for two steps
            o0 = static_cast<unsigned short>(pk & 0xFFFFu);
            o1 = static_cast<unsigned short>(pk >> 16);
          } else {
            const __half2 pk = __floats2half2_rn(y.x, y.y);
            o0 = __half_as_ushort(__low2half(pk));
            o1 = __half_as_ushort(__high2half(pk));
          }
          *reinterpret_cast<unsigned short*>(dst + (2 * j2) * (kDT * 2)) = o0;
          *reinterpret_cast<unsigned short*>(dst + (2 * j2 + 1) * (kDT * 2)) = o1;
        }
        fence_async_smem();
      }
      tc_fence_before();
      mbar_arrive_warp(smem_u32(&bars.y_staged[st]));
    };

    // one trip more than there are tiles: trip `it` writes the operand rows of tile `it` (if there is
    // one) and then finishes tile `it - 1`
    int x = x_first, c = 0, b = 0, d0 = 0;
    float Dv = 0.f;
#pragma unroll 1
    for (int it = 0; it <= ntotal; ++it) {
      if (it < ntotal) {
        if (c == 0) {
          b = x / p.ndt;
          d0 = (x - b * p.ndt) * kDT;
          Dv = (d0 + q < p.D) ? __ldg(p.Dskip + d0 + q) : 0.f;
        }
        const int st = it & 1;
        const uint32_t par = (it >> 1) & 1;
        const int t0 = c * Q, len = min(Q, p.T - t0);
        const uint32_t sidx = static_cast<uint32_t>(it) * NSLAB + grp, slot = sidx % SM::RING, ph = (sidx / SM::RING) & 1;
        // ---- (1) retention of the own 16 steps: L_j = prod_{i<=j} (1 + e^{-f_logit_i}), as pairs
        if (!mbar_wait(smem_u32(&bars.full[slot]), ph)) timeout();
        const unsigned char* sl = smem + SM::off_ring + slot * SM::slab_bytes;
        const TA* s_u = reinterpret_cast<const TA*>(sl) + q;          // [step][channel]
        const TA* s_ut = reinterpret_cast<const TA*>(sl) + q * SLAB;   // [channel][step] (time-contiguous u)
        const TG* s_fl = reinterpret_cast<const TG*>(sl + SLAB * kDT * 2) + q;
        const TG* s_il = s_fl + SLAB * kDT;
        float2 L[SLAB / 2];
        {
          float2 qv[SLAB / 2];
#pragma unroll
          for (int j2 = 0; j2 < SLAB / 2; ++j2) {
            const float2 fl2 = mul2(make_float2(ld_as_f32(s_fl, (2 * j2) * kDT), ld_as_f32(s_fl, (2 * j2 + 1) * kDT)), kk);
            qv[j2] = add2(make_float2(fast_ex2(fl2.x), fast_ex2(fl2.y)), one2);
          }
          // Steps past the end of the sequence (last chunk only) arrive as zeros from TMA: they are
          // made neutral (f = 1), so the chunk's product is the product at the last real step;
          // u = 0 keeps them out of every sum.
          const int nvalid = len - SLAB * grp;
          if (nvalid < SLAB) {
#pragma unroll
            for (int j2 = 0; j2 < SLAB / 2; ++j2) {
              if (2 * j2 >= nvalid) qv[j2].x = 1.f;
              if (2 * j2 + 1 >= nvalid) qv[j2].y = 1.f;
            }
          }
          float run = 1.f;
#pragma unroll
          for (int j2 = 0; j2 < SLAB / 2; ++j2) {
            L[j2] = mul2(make_float2(run, run), make_float2(qv[j2].x, qv[j2].x * qv[j2].y));
            run = L[j2].y;
          }
        }
        // (s_L of this stage was last read two tiles back, before those threads' arrivals on `part`,
        // which completed before the d1_full every thread has waited for in that tile's epilogue)
        s_L[st][grp][q] = L[SLAB / 2 - 1].y;
        mbar_arrive_warp(smem_u32(&bars.lprod[st][grp]));
        // ---- (2) R_t = (products of the groups before) x L_j; operand row chunks of the own slab
        // (1 / i_t does not depend on the other groups: evaluated before waiting for them)
        float2 opbv[SLAB / 2];
#pragma unroll
        for (int j2 = 0; j2 < SLAB / 2; ++j2) {
          const float2 il2 = mul2(make_float2(fmaxf(ld_as_f32(s_il, (2 * j2) * kDT), -30.f),
                                              fmaxf(ld_as_f32(s_il, (2 * j2 + 1) * kDT), -30.f)), kk);
          opbv[j2] = add2(make_float2(fast_ex2(il2.x), fast_ex2(il2.y)), one2);
        }
        float Rstart = 1.f;
        for (int g2 = 0; g2 < grp; ++g2) {
          if (!mbar_wait(smem_u32(&bars.lprod[st][g2]), par)) timeout();
          Rstart *= s_L[st][g2][q];
        }
        const float2 Rs2 = make_float2(Rstart, Rstart);
        unsigned char* a_row = smem + SM::off_AW + st * AW_BYTES + static_cast<uint32_t>(q >> 3) * SBO_AW +
                               static_cast<uint32_t>(q & 7) * 16;
        const uint32_t tP = tmem + st * TM_STAGE + lane_off + TM_P + SLAB * grp;
#pragma unroll
        for (int j8 = 0; j8 < SLAB / 8; ++j8) {
          uint32_t hi[4], lo[4], pv[8];
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const int j2 = 4 * j8 + jj;
            const float2 opb = opbv[j2];                                                   // 1 / i_t
            const float2 u2 = utm ? ld_pair_as_f32(s_ut + 2 * j2)
                                  : make_float2(ld_as_f32(s_u, (2 * j2) * kDT), ld_as_f32(s_u, (2 * j2 + 1) * kDT));
            const float2 R = mul2(Rs2, L[j2]);
            const float2 x2 = mul2(R, opb);
            const float2 r = make_float2(fast_rcp(x2.x), fast_rcp(x2.y));
            const float2 P = mul2(opb, r);                          // P_t = 1 / R_t
            pv[2 * jj] = __float_as_uint(P.x);
            pv[2 * jj + 1] = __float_as_uint(P.y);
            const float2 w = mul2(u2, mul2(mul2(R, r), R));         // u_t i_t R_t
            split_pair(w, hi[jj], lo[jj]);
          }
          *reinterpret_cast<uint4*>(a_row + (AW_W1 + 2 * grp + j8) * 128) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
          *reinterpret_cast<uint4*>(a_row + (AW_W2 + 2 * grp + j8) * 128) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
          asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(tP + 8 * j8),
                       "r"(pv[0]), "r"(pv[1]), "r"(pv[2]), "r"(pv[3]), "r"(pv[4]), "r"(pv[5]), "r"(pv[6]), "r"(pv[7]));
        }
        mbar_arrive_warp(smem_u32(&bars.empty[slot]));            // the slab has been read
        // the last group holds the whole chunk's product: the carry warps' P_Q and deep-gate decision
        // (s_Rend of the tile two back was read before that tile's acc_free, which this thread
        // waited for in that tile's epilogue)
        if (grp == NGRP - 1) s_Rend[st][q] = Rstart * L[SLAB / 2 - 1].y;
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        fence_async_smem();
        mbar_arrive_warp(smem_u32(&bars.part[st][grp]));
      }
      // ---- (3) the previous tile's outputs for the same steps
      if (it > 0) epilogue();
      if (it < ntotal) {
        e_b = b; e_d0 = d0; e_t0 = c * Q; e_len = min(Q, p.T - c * Q); e_it = it; e_Dv = Dv;
        if (++c == nchunks) {
          c = 0;
          x += x_step;
        }
      }
    }
  }
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}

}  // namespace tc3

// ------------------------------------------------------------------------------ host side
namespace {

template <typename TA, typename TG, bool UTM>
int launch_tc3_t(const FwdParams& p, const Geometry& g, const tc3::Maps& maps, cudaStream_t st) {
  const size_t smem = tc3::Smem<TG>::total;
  auto kern = tc3::fwd_tc3_kernel<TA, TG, UTM>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return static_cast<int>(e);
  // one persistent CTA per SM; channel tiles are dealt round-robin
  const int64_t grid = std::min<int64_t>(static_cast<int64_t>(g.B) * g.ndt, tmah::sm_count());
  kern<<<static_cast<unsigned>(grid), tc3::NTHREADS, smem, st>>>(p, maps);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

// Walk-along-time forward; returns -1000 if this problem cannot take it (too few channel tiles to
// fill the GPU, or shapes / strides TMA cannot describe): the caller then uses another kernel.
int launch_fwd_tc3(const FwdParams& p, const Geometry& g, int act, int gate, int bc, void* stream) {
  const bool act16 = act == NAJU_BF16 || act == NAJU_F16;
  if (!(g.N == tc3::NS && g.TC == tc3::Q && act16 && bc == NAJU_BF16 && (gate == act || gate == NAJU_F32)))
    return -1000;
  if (g.ntiles >= (1LL << 31)) return -1000;
  // (with fewer than about a quarter of the SMs busy the ticket-mode kernel, which spreads over time as
  // well, is the faster one)
  if (static_cast<int64_t>(g.B) * g.ndt * 4 < tmah::sm_count() || g.nchunks < 4) return -1000;
  tc3::Maps maps;
  const bool ok =
      (p.u_sd > 1 ? tmah::make_map_tmajor(&maps.u, p.u, act, g.B, g.T, g.D, p.u_sb, p.u_sd, tc3::SLAB, kDT)
                  : tmah::make_map(&maps.u, p.u, act, g.B, g.T, g.D, p.u_sb, p.u_st, kDT, tc3::SLAB)) &&
      tmah::make_map(&maps.fl, p.fl, gate, g.B, g.T, g.D, p.fl_sb, p.fl_st, kDT, tc3::SLAB) &&
      tmah::make_map(&maps.il, p.il, gate, g.B, g.T, g.D, p.il_sb, p.il_st, kDT, tc3::SLAB) &&
      tmah::make_map(&maps.bm, p.Bm, bc, g.B, g.T, g.N, p.bm_sb, p.bm_st, tc3::NS, tc3::Q) &&
      tmah::make_map(&maps.cm, p.Cm, bc, g.B, g.T, g.N, p.cm_sb, p.cm_st, tc3::NS, tc3::Q) &&
      tmah::make_map(&maps.y, p.y, act, g.B, g.T, g.D, static_cast<int64_t>(g.T) * g.D, g.D, kDT, tc3::Q);
  if (!ok) return -1000;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (p.u_sd > 1) {
    if (act == NAJU_BF16 && gate == NAJU_BF16) return launch_tc3_t<__nv_bfloat16, __nv_bfloat16, true>(p, g, maps, st);
    if (act == NAJU_BF16 && gate == NAJU_F32) return launch_tc3_t<__nv_bfloat16, float, true>(p, g, maps, st);
    if (act == NAJU_F16 && gate == NAJU_F16) return launch_tc3_t<__half, __half, true>(p, g, maps, st);
    if (act == NAJU_F16 && gate == NAJU_F32) return launch_tc3_t<__half, float, true>(p, g, maps, st);
  }
  if (act == NAJU_BF16 && gate == NAJU_BF16) return launch_tc3_t<__nv_bfloat16, __nv_bfloat16, false>(p, g, maps, st);
  if (act == NAJU_BF16 && gate == NAJU_F32) return launch_tc3_t<__nv_bfloat16, float, false>(p, g, maps, st);
  if (act == NAJU_F16 && gate == NAJU_F16) return launch_tc3_t<__half, __half, false>(p, g, maps, st);
  if (act == NAJU_F16 && gate == NAJU_F32) return launch_tc3_t<__half, float, false>(p, g, maps, st);
  return -1000;
}

}  // namespace naju
