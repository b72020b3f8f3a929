// Forward gated scan, chunked (state-expansion) form: persistent, TMA-fed, warp-specialised,
// tcgen05/TMEM, two threads per channel.
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
// the carry never leaves the chip.  Twenty warps in five roles, two pipeline stages (operand
// rows, shared operands and TMEM accumulators are double buffered):
//   warp 16     TMA producer: u / f_logit / i_logit in 16-step slabs through a 4-deep mbarrier
//               ring, plus the chunk's B and C rows and a second copy of u for the epilogue.
//   warps 8-15  gate warps, two threads per channel (steps 0-31 / 32-63 of the chunk; the second
//               thread first multiplies up the retention of steps 0-31 to enter step 32 with
//               the right product): sigmoids, running products, the channel's operand row
//               (K-major, no swizzle) and P_t, which goes to TMEM with tcgen05.st.
//   warps 17-18 operand builders: C | g1 | g2 and B^T of the tile with mma.sync (16x8 blocks of G dealt
//               round-robin), started as soon as the MMAs of the tile two back have read the stage.
//   warp 19     MMA issuer: one thread issues every tcgen05.mma, slab by slab as the gate warps
//               deliver, and every tcgen05.commit.
//   warps 0-7   carry/epilogue warps: warps 0-3 turn D2 into the next chunk's carry-in (registers),
//               write the checkpoint and post the carry-in row one tile ahead; all eight read
//               y_t = P_t D1[d][t] back from TMEM (lane = channel, 16 / 48 columns per thread),
//               add D_skip u_t (u is kept in shared memory for this), stage the tile in shared
//               memory and hand it to a TMA store.
// A tile whose retention product falls below 2^-80 in any channel (deep gates) cannot use the
// 1/P_t factorisation; warps 0-3 then run the exact recurrence for that tile straight from global
// memory, from the carry they hold.  Every wait is bounded.
#include <algorithm>
#include <type_traits>

#include "fwd_common.cuh"
#include "tc_common.cuh"
#include "tma_host.h"

namespace naju {
namespace tc3 {

using namespace tcx;

constexpr int Q = 64, NS = 16, SLAB = 16, NSLAB = Q / SLAB, RING = 4, NSTAGE = 2;
// NGRP gate groups of 128 threads: group g owns the steps of slabs [g * NSLAB / NGRP, (g + 1) * NSLAB / NGRP)
constexpr int NGRP = 2, SPG = NSLAB / NGRP;  // (four groups measured slower: 0.89 ms against 0.83 ms)
// NBUILD operand-builder warps share a tile's work (one warp alone takes 5.5 k cycles per tile, longer
// than the gate warps; with two the MMA issuer no longer waits for operands; four measured slower)
constexpr int NBUILD = 2;
constexpr int NHALF = 128, NGATE = NGRP * 128, NEPI = 256, NTHREADS = NEPI + NGATE + 32 * (2 + NBUILD);
constexpr int W_PROD = (NEPI + NGATE) / 32, W_BUILD = W_PROD + 1, W_MMA = W_BUILD + NBUILD;
constexpr int AW_W1 = 0, AW_W2 = 8;
constexpr uint32_t SBO_AW = 16 * 128, AW_BYTES = 16 * SBO_AW;  // operand rows [w1 64 | w2 64], per stage
constexpr int AH_H1 = 0, AH_H2 = 2;
constexpr uint32_t SBO_AH = 4 * 128, AH_BYTES = 16 * SBO_AH;   // carry-in rows [h1 16 | h2 16]
constexpr int B1_C = 0, B1_G1 = 2, B1_G2 = 10;
constexpr uint32_t SBO_B1 = 18 * 128, B1_BYTES = 8 * SBO_B1;   // rows t: [C 16 | g1 64 | g2 64]
constexpr uint32_t SBO_B2 = 8 * 128, B2_BYTES = 2 * SBO_B2;    // rows n: [B^T 64]
constexpr uint32_t BC_BYTES = Q * NS * 2;
constexpr uint32_t TM_D1 = 0, TM_D2 = 64, TM_P = 96, TM_STAGE = 160, TMEM_COLS = 512;
constexpr float kRMax = 1.0e24f;  // ~2^80
constexpr float kNegLog2e = -1.4426950408889634f;
// nanoseconds between polls for the roles that have slack (producer, builders, the epilogue warps'
// first wait of a tile); the gate warps and the MMA issuer poll without sleeping
constexpr int kRelaxProd = 100, kRelaxBuild = 100, kRelaxEpi = 64;
constexpr int EPI_A_COLS = 16;    // columns of a tile the carry warps take in the epilogue (rest: warps 4-7)

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

#ifdef NAJU_PROF
__device__ unsigned long long g_prof[48];
#define PROF_MARK(i)                                                      \
  do {                                                                    \
    if ((threadIdx.x & 127) == 0) {                                       \
      const long long now_ = clock64();                                   \
      atomicAdd(&g_prof[i], static_cast<unsigned long long>(now_ - pt_)); \
      pt_ = now_;                                                         \
    }                                                                     \
  } while (0)
#define PROF_INIT long long pt_ = clock64()
// same for the single-warp roles (lane 0 marks)
#define PROF_MARK1(i)                                                     \
  do {                                                                    \
    if ((threadIdx.x & 31) == 0) {                                        \
      const long long now_ = clock64();                                   \
      atomicAdd(&g_prof[i], static_cast<unsigned long long>(now_ - pt_)); \
      pt_ = now_;                                                         \
    }                                                                     \
  } while (0)
#else
#define PROF_MARK1(i) do {} while (0)
#define PROF_MARK(i) do {} while (0)
#define PROF_INIT do {} while (0)
#endif

struct Maps {
  CUtensorMap u, fl, il, bm, cm, y;
};

template <typename TG>
struct Smem {
  static constexpr uint32_t slab_bytes = SLAB * kDT * (2 + 2 * sizeof(TG));  // u, f_logit, i_logit
  // With 16-bit logits there is room to keep a second copy of the tile's u for the epilogue
  // (D_skip u_t); with fp32 logits the epilogue reads u from global memory instead.
  static constexpr bool kStashU = sizeof(TG) == 2;
  static constexpr uint32_t off_ring = 0;
  static constexpr uint32_t off_U = off_ring + RING * slab_bytes;                      // [NSTAGE][Q][128]
  static constexpr uint32_t off_AW = off_U + (kStashU ? NSTAGE * Q * kDT * 2 : 0);     // [NSTAGE]
  static constexpr uint32_t off_AH = off_AW + NSTAGE * AW_BYTES;
  static constexpr uint32_t off_B1 = off_AH + AH_BYTES;             // [NSTAGE]
  static constexpr uint32_t off_B2 = off_B1 + NSTAGE * B1_BYTES;    // [NSTAGE]
  static constexpr uint32_t off_bc = off_B2 + NSTAGE * B2_BYTES;    // [2 tiles][B raw | C raw]
  static constexpr uint32_t total = off_bc + 2 * 2 * BC_BYTES;
};

struct Bars {
  unsigned long long full[RING], empty[RING];   // input slabs (producer -> gate warps)
  unsigned long long u_full[NSTAGE];            // the epilogue's copy of the tile's u has landed
  unsigned long long bc_full[2], bc_empty[2];   // raw B/C rows per tile parity
  unsigned long long part[NSTAGE][NSLAB];       // operand-row chunks of one slab written (128 threads)
  unsigned long long a_full[NSTAGE];            // all gate threads done with the tile (P_t in TMEM, flags)
  unsigned long long ops_full[NSTAGE];          // builder -> MMA issuer
  unsigned long long d2_full[NSTAGE];           // D2 and the first part of D1 complete
  unsigned long long h_ready;                   // carry warps -> MMA issuer (carry-in row written)
  unsigned long long d1_full[NSTAGE];           // D1 complete (and the stage's shared operands read)
  unsigned long long stage_free[NSTAGE];        // carry/epilogue warps -> everyone upstream
};

// Exact recurrence of one tile straight from global memory (deep-gate tiles only), run by the 128
// carry threads from the carry they hold: hw / Pw = state and cumulative decay entering the chunk,
// updated to the chunk-end values (which are also written as the checkpoint).
template <typename TA, typename TG>
__device__ __noinline__ void exact_tile_from_global(const FwdParams& p, const TileCoord& tc, int tid,
                                                    float (&hw)[NS], float& Pw) {
  const TA* gu = reinterpret_cast<const TA*>(p.u) + tc.b * p.u_sb + static_cast<int64_t>(tc.t0) * p.u_st + tc.d;
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
template <typename TA, typename TG>
__global__ void __launch_bounds__(NTHREADS, 1)
fwd_tc3_kernel(const FwdParams p, const __grid_constant__ Maps maps) {
  using SM = Smem<TG>;
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ Bars bars;
  __shared__ int s_stage_deep[NSTAGE];
  __shared__ unsigned int s_tmem;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t sbase = smem_u32(smem);
  const int nchunks = p.nchunks, ctiles = p.B * p.ndt;
  const int x_first = static_cast<int>(blockIdx.x), x_step = static_cast<int>(gridDim.x);

  if (tid == 0) {
    for (int i = 0; i < RING; ++i) {
      mbar_init(smem_u32(&bars.full[i]), 1);
      mbar_init(smem_u32(&bars.empty[i]), NGATE);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars.bc_full[i]), 1);
      mbar_init(smem_u32(&bars.bc_empty[i]), NBUILD);
    }
    for (int i = 0; i < NSTAGE; ++i) {
      for (int k = 0; k < NSLAB; ++k) mbar_init(smem_u32(&bars.part[i][k]), NHALF);
      mbar_init(smem_u32(&bars.a_full[i]), NGATE);
      mbar_init(smem_u32(&bars.u_full[i]), 1);
      mbar_init(smem_u32(&bars.ops_full[i]), NBUILD);
      mbar_init(smem_u32(&bars.d2_full[i]), 1);
      mbar_init(smem_u32(&bars.stage_free[i]), NEPI);
    }
    mbar_init(smem_u32(&bars.h_ready), NHALF);
    for (int i = 0; i < NSTAGE; ++i) mbar_init(smem_u32(&bars.d1_full[i]), 1);
    mbar_init_fence();
    if (blockIdx.x == 0) {
      atomicOr(p.fwd_form, 1);  // tell the backward how the forward ran
      p.hdr->form = NAJU_FORM_TC_WALK;
    }
  }
  if (warp == 0) tmem_alloc(smem_u32(&s_tmem), TMEM_COLS);
  // the upper triangle of g1/g2 is never written again: clear the shared operands once
  for (uint32_t i = tid * 16; i < NSTAGE * (B1_BYTES + B2_BYTES); i += NTHREADS * 16)
    *reinterpret_cast<uint4*>(smem + SM::off_B1 + i) = make_uint4(0, 0, 0, 0);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;
  auto timeout = [&]() { atomicOr(&p.hdr->status, NAJU_ST_MMA_TIMEOUT); };

  if (warp == W_PROD) {
    // ===================================================================== TMA producer
    if (lane == 0) {
      uint32_t slab = 0;
      int it = 0;
      // The epilogue's copy of tile j's u goes to the stage buffer once the tile two back has left
      // it; it is requested one tile late, where waiting for that cannot hold up any other load.
      int pb = 0, pd0 = 0, pt0 = 0;
      auto load_u_copy = [&](int j) {
        if constexpr (SM::kStashU) {
          const int st = j & 1;
          if (j >= NSTAGE && !mbar_wait_relaxed<kRelaxProd>(smem_u32(&bars.stage_free[st]), ((j >> 1) & 1) ^ 1)) timeout();
          const uint32_t bar = smem_u32(&bars.u_full[st]);
          mbar_arrive_expect_tx(bar, Q * kDT * 2);
          for (int k = 0; k < NSLAB; ++k)
            tma_load_3d(sbase + SM::off_U + st * Q * kDT * 2 + k * SLAB * kDT * 2, &maps.u, pd0, pt0 + k * SLAB, pb, bar);
        }
      };
      for (int x = x_first; x < ctiles; x += x_step) {
        const int b = x / p.ndt, d0 = (x - b * p.ndt) * kDT;
        for (int c = 0; c < nchunks; ++c, ++it) {
          const int t0 = c * Q;
          if (it >= 1) load_u_copy(it - 1);
          pb = b;
          pd0 = d0;
          pt0 = t0;
          if (it >= 2 && !mbar_wait_relaxed<kRelaxProd>(smem_u32(&bars.bc_empty[it & 1]), ((it >> 1) & 1) ^ 1)) timeout();
          {
            const uint32_t bar = smem_u32(&bars.bc_full[it & 1]);
            const uint32_t dst = sbase + SM::off_bc + (it & 1) * 2 * BC_BYTES;
            mbar_arrive_expect_tx(bar, 2 * BC_BYTES);
            tma_load_3d(dst, &maps.bm, 0, t0, b, bar);
            tma_load_3d(dst + BC_BYTES, &maps.cm, 0, t0, b, bar);
          }
          for (int k = 0; k < NSLAB; ++k, ++slab) {
            const uint32_t slot = slab % RING, ph = (slab / RING) & 1;
            if (slab >= RING && !mbar_wait_relaxed<kRelaxProd>(smem_u32(&bars.empty[slot]), ph ^ 1)) timeout();
            const uint32_t bar = smem_u32(&bars.full[slot]);
            const uint32_t dst = sbase + SM::off_ring + slot * SM::slab_bytes;
            mbar_arrive_expect_tx(bar, SM::slab_bytes);
            tma_load_3d(dst, &maps.u, d0, t0 + k * SLAB, b, bar);
            tma_load_3d(dst + SLAB * kDT * 2, &maps.fl, d0, t0 + k * SLAB, b, bar);
            tma_load_3d(dst + SLAB * kDT * (2 + sizeof(TG)), &maps.il, d0, t0 + k * SLAB, b, bar);
          }
        }
      }
      if (it >= 1) load_u_copy(it - 1);
    }
  } else if (warp >= W_BUILD && warp < W_BUILD + NBUILD) {
    // ===================================================================== operand builders
    const int g = lane >> 2, t4 = lane & 3;
    const int bw = warp - W_BUILD, blane = bw * 32 + lane;
    int it = 0;
    PROF_INIT;
    for (int x = x_first; x < ctiles; x += x_step) {
      for (int c = 0; c < nchunks; ++c, ++it) {
        const int st = it & 1;
        if (!mbar_wait_relaxed<kRelaxBuild>(smem_u32(&bars.bc_full[st]), (it >> 1) & 1)) timeout();
        // stage st: the MMAs of the tile two back must have read B1 / B2 (its epilogue may still run)
        if (it >= NSTAGE && !mbar_wait_relaxed<kRelaxBuild>(smem_u32(&bars.d1_full[st]), ((it >> 1) & 1) ^ 1)) timeout();
        PROF_MARK1(40);
        unsigned char* s_B1 = smem + SM::off_B1 + st * B1_BYTES;
        unsigned char* s_B2 = smem + SM::off_B2 + st * B2_BYTES;
        const __nv_bfloat16* Braw = reinterpret_cast<const __nv_bfloat16*>(smem + SM::off_bc + st * 2 * BC_BYTES);
        const __nv_bfloat16* Craw = Braw + Q * NS;
        for (int e = blane; e < Q * 2; e += 32 * NBUILD) {  // C columns of B1: 32 bytes per row
          const int t = e >> 1, half = e & 1;
          *reinterpret_cast<uint4*>(s_B1 + op_off16(t, B1_C * 8 + half * 8, SBO_B1)) =
              *reinterpret_cast<const uint4*>(Craw + t * NS + half * 8);
        }
        for (int e = blane; e < NS * (Q / 8); e += 32 * NBUILD) {  // B2 = B^T: (row n, eight columns s) per store
          const int n = e % NS, s8 = e / NS;
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t lo = *reinterpret_cast<const unsigned short*>(Braw + (8 * s8 + 2 * j) * NS + n);
            const uint32_t hi = *reinterpret_cast<const unsigned short*>(Braw + (8 * s8 + 2 * j + 1) * NS + n);
            w[j] = lo | (hi << 16);
          }
          *reinterpret_cast<uint4*>(s_B2 + op_off16(n, 8 * s8, SBO_B2)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
#pragma unroll 1
        for (int mt = 0; mt < Q / 16; ++mt) {  // G = tril(C B^T) in two bf16 terms
          const int r0 = 16 * mt + g, r1 = r0 + 8;
          const uint32_t a0 = *reinterpret_cast<const uint32_t*>(Craw + r0 * NS + 2 * t4);
          const uint32_t a1 = *reinterpret_cast<const uint32_t*>(Craw + r1 * NS + 2 * t4);
          const uint32_t a2 = *reinterpret_cast<const uint32_t*>(Craw + r0 * NS + 2 * t4 + 8);
          const uint32_t a3 = *reinterpret_cast<const uint32_t*>(Craw + r1 * NS + 2 * t4 + 8);
          for (int nt = 0; nt <= 2 * mt + 1; ++nt) {
            if (((mt * (mt + 1) + nt) % NBUILD) != bw) continue;  // 16x8 blocks dealt round-robin to the builder warps
            float c4[4] = {0.f, 0.f, 0.f, 0.f};
            const uint32_t b0 = *reinterpret_cast<const uint32_t*>(Braw + (8 * nt + g) * NS + 2 * t4);
            const uint32_t b1 = *reinterpret_cast<const uint32_t*>(Braw + (8 * nt + g) * NS + 2 * t4 + 8);
            mma_bf16_16x8x16(c4, a0, a1, a2, a3, b0, b1);
            const int s0 = 8 * nt + 2 * t4;
            uint32_t hi, lo;
            split_bf16x2(s0 <= r0 ? c4[0] : 0.f, s0 + 1 <= r0 ? c4[1] : 0.f, hi, lo);
            *reinterpret_cast<uint32_t*>(s_B1 + op_off16(r0, B1_G1 * 8 + s0, SBO_B1)) = hi;
            *reinterpret_cast<uint32_t*>(s_B1 + op_off16(r0, B1_G2 * 8 + s0, SBO_B1)) = lo;
            split_bf16x2(s0 <= r1 ? c4[2] : 0.f, s0 + 1 <= r1 ? c4[3] : 0.f, hi, lo);
            *reinterpret_cast<uint32_t*>(s_B1 + op_off16(r1, B1_G1 * 8 + s0, SBO_B1)) = hi;
            *reinterpret_cast<uint32_t*>(s_B1 + op_off16(r1, B1_G2 * 8 + s0, SBO_B1)) = lo;
          }
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(smem_u32(&bars.ops_full[st]));
          mbar_arrive(smem_u32(&bars.bc_empty[st]));
        }
        PROF_MARK1(41);
      }
    }
  } else if (warp == W_MMA) {
    // ===================================================================== MMA issuer
    if (lane == 0) {
      const uint32_t id16 = umma_idesc(128, NS, 1), id64 = umma_idesc(128, Q, 1);
      // operand addresses are fixed: build the descriptors once, offset the address field per use
      const uint64_t dAW0 = umma_desc(sbase + SM::off_AW, 128, SBO_AW), dAH = umma_desc(sbase + SM::off_AH, 128, SBO_AH);
      const uint64_t dB10 = umma_desc(sbase + SM::off_B1, 128, SBO_B1), dB20 = umma_desc(sbase + SM::off_B2, 128, SBO_B2);
      auto off = [](uint32_t bytes) { return static_cast<uint64_t>(bytes >> 4); };
      PROF_INIT;
      int it = 0;
      for (int x = x_first; x < ctiles; x += x_step) {
        for (int c = 0; c < nchunks; ++c, ++it) {
          const int st = it & 1;
          const uint32_t par = (it >> 1) & 1;
          const uint64_t dAW = dAW0 + off(st * AW_BYTES), dB1 = dB10 + off(st * B1_BYTES), dB2 = dB20 + off(st * B2_BYTES);
          const uint32_t tst = tmem + st * TM_STAGE;
          if (!mbar_wait(smem_u32(&bars.ops_full[st]), par)) timeout();
          PROF_MARK1(32);
#pragma unroll 1
          for (int ks = 0; ks < NSLAB; ++ks) {
            // the time contractions of slab ks run while the gate warps are still on the other slabs
            if (!mbar_wait(smem_u32(&bars.part[st][ks]), par)) timeout();
            tc_fence_after();
            const uint64_t w1 = dAW + off((AW_W1 + 2 * ks) * 128), w2 = dAW + off((AW_W2 + 2 * ks) * 128);
            umma_bf16(tst + TM_D2, w1, dB2 + off(2 * ks * 128), id16, ks > 0);   // D2 += (w1 + w2) . B^T
            umma_bf16(tst + TM_D2, w2, dB2 + off(2 * ks * 128), id16, 1u);
            umma_bf16(tst + TM_D1, w1, dB1 + off((B1_G1 + 2 * ks) * 128), id64, ks > 0);  // D1 += w1.g1 + w1.g2 + w2.g1
            umma_bf16(tst + TM_D1, w1, dB1 + off((B1_G2 + 2 * ks) * 128), id64, 1u);
            umma_bf16(tst + TM_D1, w2, dB1 + off((B1_G1 + 2 * ks) * 128), id64, 1u);
          }
          // a deep-gate tile is decided only now (all gate threads done): its accumulators are junk
          // and are simply not read; one carry-in phase per tile keeps the phase counts aligned
          PROF_MARK1(33);
          if (!mbar_wait(smem_u32(&bars.a_full[st]), par)) timeout();
          umma_commit(smem_u32(&bars.d2_full[st]));
          PROF_MARK1(34);
          if (!mbar_wait(smem_u32(&bars.h_ready), it & 1)) timeout();
          PROF_MARK1(35);
          if (!s_stage_deep[st]) {
            tc_fence_after();
            umma_bf16(tst + TM_D1, dAH + off(AH_H1 * 128), dB1 + off(B1_C * 128), id64, 1u);  // D1 += (h1 + h2) . C
            umma_bf16(tst + TM_D1, dAH + off(AH_H2 * 128), dB1 + off(B1_C * 128), id64, 1u);
          }
          umma_commit(smem_u32(&bars.d1_full[st]));
          PROF_MARK1(36);
        }
      }
    }
  } else if (warp >= 8) {
    // ===================================================================== gate warps
    const int half = (warp - 8) >> 2;      // gate group: which slabs of every chunk this thread evaluates
    const int q = tid & (kDT - 1);         // channel within the tile
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    uint32_t slab = 0;
    int it = 0;
    PROF_INIT;
    for (int x = x_first; x < ctiles; x += x_step) {
      for (int c = 0; c < nchunks; ++c, ++it) {
        const int st = it & 1;
        if (it >= NSTAGE && !mbar_wait(smem_u32(&bars.stage_free[st]), ((it >> 1) & 1) ^ 1)) timeout();
        PROF_MARK(16 + 8 * half);
        tc_fence_after();
        unsigned char* a_row = smem + SM::off_AW + st * AW_BYTES + static_cast<uint32_t>(q >> 3) * SBO_AW +
                               static_cast<uint32_t>(q & 7) * 16;
        const uint32_t tP = tmem + st * TM_STAGE + TM_P + lane_off;
        // Steps past the end of the sequence (last chunk only) arrive as zeros from TMA: u = 0 keeps
        // them out of every sum, and the carry warps take the decay product at the last real step.
        float R = 1.f;
#pragma unroll 1
        for (int k = 0; k < NSLAB; ++k) {
          const uint32_t sidx = slab + k, slot = sidx % RING, ph = (sidx / RING) & 1;
          const bool mine = (k / SPG) == half;
          // (every thread waits for the slab before releasing it, needed or not: an arrival must
          // not reach the empty barrier before its previous phase has completed)
#ifdef NAJU_PROF
          const long long tw_ = clock64();
#endif
          if (!mbar_wait(smem_u32(&bars.full[slot]), ph)) timeout();
#ifdef NAJU_PROF
          if ((threadIdx.x & 127) == 0) atomicAdd(&g_prof[16 + 8 * half + 3], static_cast<unsigned long long>(clock64() - tw_));
#endif
          const unsigned char* sl = smem + SM::off_ring + slot * SM::slab_bytes;
          const TA* s_u = reinterpret_cast<const TA*>(sl) + q;
          const TG* s_fl = reinterpret_cast<const TG*>(sl + SLAB * kDT * 2) + q;
          const TG* s_il = s_fl + SLAB * kDT;
          if (!mine) {
            if (k / SPG < half) {
              // slabs before this group's: retention products only.  The sixteen factors are
              // independent: multiply them as a tree, not as a chain.
              float fac[SLAB];
#pragma unroll
              for (int tl = 0; tl < SLAB; ++tl) fac[tl] = 1.f + fast_ex2(ld_as_f32(s_fl, tl * kDT) * kNegLog2e);
#pragma unroll
              for (int w = SLAB / 2; w >= 1; w >>= 1)
#pragma unroll
                for (int i = 0; i < w; ++i) fac[i] *= fac[i + w];
              R *= fac[0];
            }
            mbar_arrive(smem_u32(&bars.empty[slot]));
            continue;
          }
#pragma unroll 1
          for (int j8 = 0; j8 < SLAB / 8; ++j8) {  // (loops are kept rolled: five roles share the instruction cache)
            float wv[8];
            uint32_t pv[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int tl = 8 * j8 + j;
              const float flv = ld_as_f32(s_fl, tl * kDT);
              const float ilv = fmaxf(ld_as_f32(s_il, tl * kDT), -30.f);
              const float uv = ld_as_f32(s_u, tl * kDT);
              const float a = fast_ex2(flv * kNegLog2e);
              const float opb = 1.f + fast_ex2(ilv * kNegLog2e);  // 1/i
              R *= 1.f + a;
              const float r = fast_rcp(R * opb);
              pv[j] = __float_as_uint(opb * r);                   // P_t = 1/R_t
              wv[j] = uv * (R * r) * R;                           // u * i * R
            }
            uint32_t h0, h1, h2, h3, l0, l1, l2, l3;
            split_bf16x2(wv[0], wv[1], h0, l0);
            split_bf16x2(wv[2], wv[3], h1, l1);
            split_bf16x2(wv[4], wv[5], h2, l2);
            split_bf16x2(wv[6], wv[7], h3, l3);
            const int ch = k * (SLAB / 8) + j8;
            *reinterpret_cast<uint4*>(a_row + (AW_W1 + ch) * 128) = make_uint4(h0, h1, h2, h3);
            *reinterpret_cast<uint4*>(a_row + (AW_W2 + ch) * 128) = make_uint4(l0, l1, l2, l3);
            asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(tP + 8 * ch),
                         "r"(pv[0]), "r"(pv[1]), "r"(pv[2]), "r"(pv[3]), "r"(pv[4]), "r"(pv[5]), "r"(pv[6]), "r"(pv[7])
                         : "memory");
          }
          mbar_arrive(smem_u32(&bars.empty[slot]));
          fence_async_smem();
          mbar_arrive(smem_u32(&bars.part[st][k]));
        }
        slab += NSLAB;
        PROF_MARK(16 + 8 * half + 1);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        const bool deep = half == NGRP - 1 && !(R < kRMax);  // the last group holds the whole chunk's product
        const bool any_deep = bar_or<2, NGATE>(deep);
        if (tid == 8 * 32) s_stage_deep[st] = any_deep ? 1 : 0;
        tc_fence_before();
        mbar_arrive(smem_u32(&bars.a_full[st]));
        PROF_MARK(16 + 8 * half + 2);
      }
    }
  } else {
    // ===================================================================== carry / epilogue warps
    const int half = warp >> 2;           // 0: carry + first EPI_A_COLS columns, 1: the other columns
    const int q = tid & (kDT - 1);
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    unsigned char* h_row = smem + SM::off_AH + static_cast<uint32_t>(q >> 3) * SBO_AH + static_cast<uint32_t>(q & 7) * 16;
    auto write_h_row = [&](const float (&hv)[NS]) {
      uint32_t hi[8], lo[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) split_bf16x2(hv[2 * k], hv[2 * k + 1], hi[k], lo[k]);
      *reinterpret_cast<uint4*>(h_row + (AH_H1 + 0) * 128) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
      *reinterpret_cast<uint4*>(h_row + (AH_H1 + 1) * 128) = make_uint4(hi[4], hi[5], hi[6], hi[7]);
      *reinterpret_cast<uint4*>(h_row + (AH_H2 + 0) * 128) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
      *reinterpret_cast<uint4*>(h_row + (AH_H2 + 1) * 128) = make_uint4(lo[4], lo[5], lo[6], lo[7]);
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(smem_u32(&bars.h_ready));
    };
    // state / cumulative decay entering the current chunk (first half only)
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
    if (half == 0 && x_first < ctiles) {
      load_h0(x_first);
      write_h_row(hc);
    }
    int it = 0;
    PROF_INIT;
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
      const float Dv = tcd.d_ok ? __ldg(p.Dskip + tcd.d) : 0.f;
      for (int c = 0; c < nchunks; ++c, ++it) {
        const int st = it & 1;
        if (!mbar_wait_relaxed<kRelaxEpi>(smem_u32(&bars.d2_full[st]), (it >> 1) & 1)) timeout();
        PROF_MARK(8 * half);
        tcd.c = c;
        tcd.tile = static_cast<int64_t>(c) * ctiles + x;
        tcd.t0 = c * Q;
        tcd.len = min(Q, p.T - tcd.t0);
        const int len = tcd.len;
        const bool deep = s_stage_deep[st] != 0;
        tc_fence_after();
        const uint32_t trow = tmem + st * TM_STAGE + lane_off;
        if (half == 0) {
          if (deep) {
            if (q == 0) atomicOr(p.fwd_form, 2);
            exact_tile_from_global<TA, TG>(p, tcd, q, hc, Pc);
          } else {
            // chunk aggregate from D2: chunk-end state = next carry-in = checkpoint.  The decay
            // product of the chunk is P at its last real step.
            uint32_t sr[16], pl[1];
            tmem_ld16_async(trow + TM_D2, sr);
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(pl[0]) : "r"(trow + TM_P + len - 1) : "memory");
            tmem_ld_wait16(sr);
            asm volatile("" : "+r"(pl[0])::"memory");
            const float P = __uint_as_float(pl[0]);
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
        }
        PROF_MARK(8 * half + 1);
        if (!mbar_wait(smem_u32(&bars.d1_full[st]), (it >> 1) & 1)) timeout();
        PROF_MARK(8 * half + 2);
        tc_fence_after();
        if (half == 0) {
          // the last MMA of this tile has read the carry-in row: post the next tile's row now
          if (c + 1 < nchunks) {
            write_h_row(hc);
          } else if (x + x_step < ctiles) {
            load_h0(x + x_step);
            write_h_row(hc);
          }
        }
        PROF_MARK(8 * half + 3);
        // ---- epilogue: y_t = P_t D1[d][t] + D_skip u_t, staged in the (now dead) operand rows of this
        // stage (step t -> 256 contiguous bytes), written out with 16-byte stores
        unsigned char* ystage = smem + SM::off_AW + st * AW_BYTES;
        if (!deep) {
          const TA* s_u = reinterpret_cast<const TA*>(smem + SM::off_U + st * Q * kDT * 2) + q;
          const TA* gu = reinterpret_cast<const TA*>(p.u) + tcd.b * p.u_sb + static_cast<int64_t>(tcd.t0) * p.u_st + tcd.d;
          if constexpr (SM::kStashU) {
            if (!mbar_wait(smem_u32(&bars.u_full[st]), (it >> 1) & 1)) timeout();
          }
          const int c_lo = half ? EPI_A_COLS : 0;
          const int nblk = half ? (Q - EPI_A_COLS) / 8 : EPI_A_COLS / 8;
          uint32_t vA[8], pA[8], vB[8], pB[8];
          auto emit8 = [&](int col, const uint32_t (&v)[8], const uint32_t (&pt)[8]) {
            unsigned char* dst = ystage + (col >> 3) * SBO_AW + q * 2;  // (col is a multiple of 8)
#pragma unroll
            for (int k = 0; k < 8; k += 2) {
              const int t = col + k;
              float y0 = __uint_as_float(pt[k]) * __uint_as_float(v[k]);
              float y1 = __uint_as_float(pt[k + 1]) * __uint_as_float(v[k + 1]);
              if (Dv != 0.f) {
                if constexpr (SM::kStashU) {  // (u past the end of the sequence is zero)
                  y0 = fmaf(Dv, ld_as_f32(s_u, t * kDT), y0);
                  y1 = fmaf(Dv, ld_as_f32(s_u, (t + 1) * kDT), y1);
                } else {
                  if (t < len) y0 = fmaf(Dv, to_f32(gu[static_cast<int64_t>(t) * p.u_st]), y0);
                  if (t + 1 < len) y1 = fmaf(Dv, to_f32(gu[static_cast<int64_t>(t + 1) * p.u_st]), y1);
                }
              }
              unsigned short o0, o1;
              if constexpr (std::is_same<TA, __nv_bfloat16>::value) {
                const uint32_t pk = pack_bf16x2(y0, y1);  // one conversion for two steps
                o0 = static_cast<unsigned short>(pk & 0xFFFFu);
                o1 = static_cast<unsigned short>(pk >> 16);
              } else {
                const __half2 pk = __floats2half2_rn(y0, y1);
                o0 = __half_as_ushort(__low2half(pk));
                o1 = __half_as_ushort(__high2half(pk));
              }
              *reinterpret_cast<unsigned short*>(dst + k * 256) = o0;
              *reinterpret_cast<unsigned short*>(dst + (k + 1) * 256) = o1;
            }
          };
          tmem_ld8_async(trow + TM_D1 + c_lo, vA);
          tmem_ld8_async(trow + TM_P + c_lo, pA);
          tmem_ld_wait8(vA, pA);
#pragma unroll 1
          for (int blk = 0; blk < nblk; blk += 2) {  // two eight-column blocks per trip, loads one block ahead
            const int col = c_lo + 8 * blk;
            tmem_ld8_async(trow + TM_D1 + col + 8, vB);
            tmem_ld8_async(trow + TM_P + col + 8, pB);
            emit8(col, vA, pA);
            tmem_ld_wait8(vB, pB);
            if (blk + 2 < nblk) {
              tmem_ld8_async(trow + TM_D1 + col + 16, vA);
              tmem_ld8_async(trow + TM_P + col + 16, pA);
            }
            emit8(col + 8, vB, pB);
            if (blk + 2 < nblk) tmem_ld_wait8(vA, pA);
          }
        }
        PROF_MARK(8 * half + 4);
        fence_async_smem();
        tc_fence_before();
        bar_sync<1, NEPI>();
        PROF_MARK(8 * half + 5);
        if (!deep && tid == 0) {
          // the staged tile leaves by TMA (steps past T and channels past D are clipped); the stage
          // is released once the store has read it
          tma_store_3d(&maps.y, tcd.d0, tcd.t0, tcd.b, smem_u32(ystage));
          tma_store_commit();
          tma_store_wait_read();
        }
        mbar_arrive(smem_u32(&bars.stage_free[st]));
        PROF_MARK(8 * half + 6);
      }
    }
  }
  if (tid == 0) tma_store_wait_all();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}

}  // namespace tc3

#ifdef NAJU_PROF
}  // namespace naju
extern "C" int naju_b200_debug_prof3(unsigned long long* out48, int reset) {
  if (reset) {
    unsigned long long z[48] = {};
    return static_cast<int>(cudaMemcpyToSymbol(naju::tc3::g_prof, z, sizeof(z)));
  }
  return static_cast<int>(cudaMemcpyFromSymbol(out48, naju::tc3::g_prof, 48 * sizeof(unsigned long long)));
}
namespace naju {
#endif

// ------------------------------------------------------------------------------ host side
namespace {

template <typename TA, typename TG>
int launch_tc3_t(const FwdParams& p, const Geometry& g, const tc3::Maps& maps, cudaStream_t st) {
  const size_t smem = tc3::Smem<TG>::total;
  auto kern = tc3::fwd_tc3_kernel<TA, TG>;
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
  // (with fewer than about a third of the SMs busy the ticket-mode kernel, which spreads over time as
  // well, is the faster one)
  if (static_cast<int64_t>(g.B) * g.ndt * 3 < tmah::sm_count() || g.nchunks < 4) return -1000;
  tc3::Maps maps;
  const bool ok =
      tmah::make_map(&maps.u, p.u, act, g.B, g.T, g.D, p.u_sb, p.u_st, kDT, tc3::SLAB) &&
      tmah::make_map(&maps.fl, p.fl, gate, g.B, g.T, g.D, p.fl_sb, p.fl_st, kDT, tc3::SLAB) &&
      tmah::make_map(&maps.il, p.il, gate, g.B, g.T, g.D, p.il_sb, p.il_st, kDT, tc3::SLAB) &&
      tmah::make_map(&maps.bm, p.Bm, bc, g.B, g.T, g.N, p.bm_sb, p.bm_st, tc3::NS, tc3::Q) &&
      tmah::make_map(&maps.cm, p.Cm, bc, g.B, g.T, g.N, p.cm_sb, p.cm_st, tc3::NS, tc3::Q) &&
      tmah::make_map(&maps.y, p.y, act, g.B, g.T, g.D, static_cast<int64_t>(g.T) * g.D, g.D, kDT, tc3::Q);
  if (!ok) return -1000;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (act == NAJU_BF16 && gate == NAJU_BF16) return launch_tc3_t<__nv_bfloat16, __nv_bfloat16>(p, g, maps, st);
  if (act == NAJU_BF16 && gate == NAJU_F32) return launch_tc3_t<__nv_bfloat16, float>(p, g, maps, st);
  if (act == NAJU_F16 && gate == NAJU_F16) return launch_tc3_t<__half, __half>(p, g, maps, st);
  if (act == NAJU_F16 && gate == NAJU_F32) return launch_tc3_t<__half, float>(p, g, maps, st);
  return -1000;
}

}  // namespace naju
