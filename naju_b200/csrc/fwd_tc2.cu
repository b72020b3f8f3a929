// Forward gated scan, chunked (state-expansion) form: persistent, TMA-fed, tcgen05/TMEM.
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
// Structure: persistent CTAs (2 per SM), six warps each:
//   warps 0-3  thread = channel.  Gates, running products and the A-operand row of their channel
//              (K-major, no swizzle); MMA issue by one elected thread; carry across chunks by the
//              bounded decoupled look-back; epilogue y_t = P_t D1[d][t] read back from TMEM
//              (lane = channel) and stored straight to global.
//   warp 4     TMA producer: takes tile tickets (time-major, so a chunk's predecessor is always
//              already owned by a running CTA) and streams u / f_logit / i_logit in 16-step slabs
//              through a 3-deep mbarrier ring, plus the chunk's B and C rows.
//   warp 5     builds the shared operands of the tile (C | g1 | g2 and B^T) with mma.sync while
//              warps 0-3 evaluate the gates.
// A tile whose retention product falls below 2^-80 in any channel (deep gates) cannot use the
// 1/P_t factorisation; warps 0-3 then run the exact two-pass recurrence for that tile straight
// from global memory.  Every wait (mbarrier, look-back flag) is bounded.
#include <algorithm>

#include "fwd_common.cuh"
#include "tc_common.cuh"

namespace naju {
namespace tc2 {

using namespace tcx;

constexpr int Q = 64, NS = 16, SLAB = 16, NSLAB = Q / SLAB, RING = 3;
constexpr int NCOMPUTE = 128, NTHREADS = 192;
// A operand row (bf16): [h1 16 | h2 16 | w1 64 | w2 64] = 20 chunks of 8 elements
constexpr int A_CH = 20, A_H1 = 0, A_H2 = 2, A_W1 = 4, A_W2 = 12;
constexpr uint32_t SBO_A = A_CH * 128, A_BYTES = 16 * SBO_A;  // 40960
// B1 operand row t (bf16): [C 16 | g1 64 | g2 64] = 18 chunks
constexpr int B1_CH = 18, B1_C = 0, B1_G1 = 2, B1_G2 = 10;
constexpr uint32_t SBO_B1 = B1_CH * 128, B1_BYTES = 8 * SBO_B1;  // 18432
// B2 operand row n (bf16): [B^T 64] = 8 chunks
constexpr uint32_t SBO_B2 = 8 * 128, B2_BYTES = 2 * SBO_B2;  // 2048
constexpr uint32_t BC_BYTES = Q * NS * 2;                      // one raw B (or C) tile, bf16
constexpr uint32_t TMEM_COLS = 128;                            // D1 [0,64), D2 [64,80)
constexpr float kRMax = 1.0e24f;                               // ~2^80
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

#ifdef NAJU_PROF
__device__ unsigned long long g_prof[16];
#define PROF_MARK(i)                                                     \
  do {                                                                   \
    if (tid == 0) {                                                      \
      const long long now_ = clock64();                                  \
      atomicAdd(&g_prof[i], static_cast<unsigned long long>(now_ - pt_)); \
      pt_ = now_;                                                        \
    }                                                                    \
  } while (0)
#define PROF_INIT long long pt_ = clock64()
#else
#define PROF_MARK(i) do {} while (0)
#define PROF_INIT do {} while (0)
#endif

struct Maps {
  CUtensorMap u, fl, il, bm, cm;
};

template <typename TG>
struct Smem {
  static constexpr uint32_t slab_bytes = SLAB * kDT * (2 + 2 * sizeof(TG));
  static constexpr uint32_t off_ring = 0;
  static constexpr uint32_t off_A = off_ring + RING * slab_bytes;
  static constexpr uint32_t off_B1 = off_A + A_BYTES;
  static constexpr uint32_t off_B2 = off_B1 + B1_BYTES;
  static constexpr uint32_t off_bc = off_B2 + B2_BYTES;  // [2 tiles][B raw | C raw]
  static constexpr uint32_t total = off_bc + 2 * 2 * BC_BYTES;
};

struct Bars {
  unsigned long long full[RING], empty[RING];  // input slabs
  unsigned long long bc_full[2], bc_empty[2];  // raw B/C rows per tile parity
  unsigned long long ops_full, ops_empty;      // shared MMA operands built / released
  unsigned long long d2, d1;                   // tcgen05.commit targets
};

// exact two-pass recurrence of one tile straight from global memory (deep-gate tiles only)
template <typename TA, typename TG>
__device__ __noinline__ void exact_tile_from_global(const FwdParams& p, const TileCoord& tc, int tid) {
  const TA* gu = reinterpret_cast<const TA*>(p.u) + tc.b * p.u_sb + static_cast<int64_t>(tc.t0) * p.u_st + tc.d;
  const TG* gf = reinterpret_cast<const TG*>(p.fl) + tc.b * p.fl_sb + static_cast<int64_t>(tc.t0) * p.fl_st + tc.d;
  const TG* gi = reinterpret_cast<const TG*>(p.il) + tc.b * p.il_sb + static_cast<int64_t>(tc.t0) * p.il_st + tc.d;
  const int64_t bbase = tc.b * p.bm_sb + static_cast<int64_t>(tc.t0) * p.bm_st;
  const int64_t cbase = tc.b * p.cm_sb + static_cast<int64_t>(tc.t0) * p.cm_st;
  float x[NS], h[NS];
  float P = 1.f, Pin;
#pragma unroll
  for (int n = 0; n < NS; ++n) x[n] = 0.f;
  for (int t = 0; t < tc.len; ++t) {
    float f = 1.f, w = 0.f;
    if (tc.d_ok) {
      f = sigmoid_f(to_f32(gf[t * p.fl_st]));
      w = sigmoid_f(to_f32(gi[t * p.il_st])) * to_f32(gu[t * p.u_st]);
    }
    P *= f;
#pragma unroll
    for (int n = 0; n < NS; ++n)
      x[n] = fmaf(f, x[n], w * (n < p.N ? load_dyn(p.Bm, p.bc_dtype, bbase + t * p.bm_st + n) : 0.f));
  }
  carry_lookback<NS, true>(p, tc, tid, x, P, h, Pin);
  const float Dv = tc.d_ok ? p.Dskip[tc.d] : 0.f;
  TA* gy = reinterpret_cast<TA*>(p.y) + (static_cast<int64_t>(tc.b) * p.T + tc.t0) * p.D + tc.d;
  for (int t = 0; t < tc.len; ++t) {
    float f = 1.f, w = 0.f, ut = 0.f;
    if (tc.d_ok) {
      ut = to_f32(gu[t * p.u_st]);
      f = sigmoid_f(to_f32(gf[t * p.fl_st]));
      w = sigmoid_f(to_f32(gi[t * p.il_st])) * ut;
    }
    float acc = 0.f;
#pragma unroll
    for (int n = 0; n < NS; ++n) {
      const float bv = n < p.N ? load_dyn(p.Bm, p.bc_dtype, bbase + t * p.bm_st + n) : 0.f;
      const float cv = n < p.N ? load_dyn(p.Cm, p.bc_dtype, cbase + t * p.cm_st + n) : 0.f;
      h[n] = fmaf(f, h[n], w * bv);
      acc = fmaf(cv, h[n], acc);
    }
    if (tc.d_ok) gy[static_cast<int64_t>(t) * p.D] = from_f32<TA>(fmaf(Dv, ut, acc));
  }
  write_final<NS>(p, tc, h, P * Pin);
}

template <typename TA, typename TG>
__global__ void __launch_bounds__(NTHREADS, 2)
fwd_tc2_kernel(const FwdParams p, const __grid_constant__ Maps maps, const int ntiles) {
  using SM = Smem<TG>;
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ Bars bars;
  __shared__ int s_tile[2];
  __shared__ unsigned int s_tmem;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t sbase = smem_u32(smem);

  if (tid == 0) {
    for (int i = 0; i < RING; ++i) {
      mbar_init(smem_u32(&bars.full[i]), 1);
      mbar_init(smem_u32(&bars.empty[i]), NCOMPUTE);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars.bc_full[i]), 1);
      mbar_init(smem_u32(&bars.bc_empty[i]), 1);
    }
    mbar_init(smem_u32(&bars.ops_full), 1);
    mbar_init(smem_u32(&bars.ops_empty), 1);
    mbar_init(smem_u32(&bars.d2), 1);
    mbar_init(smem_u32(&bars.d1), 1);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(smem_u32(&s_tmem), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;

  if (warp == 4) {
    // ===================================================================== TMA producer
    uint32_t slab = 0;  // running slab counter across tiles
    for (int it = 0;; ++it) {
      int tile = 0;
      if (lane == 0) {
        const unsigned ticket = atomicAdd(&p.hdr->ticket, 1u);
        tile = ticket < static_cast<unsigned>(ntiles) ? static_cast<int>(ticket) : -1;
        // s_tile[it & 1] was last read for tile it-2, whose slabs were all released before the
        // ring let the producer get this far (it is at most RING < NSLAB slabs ahead).
        const uint32_t slot0 = slab % RING, ph0 = (slab / RING) & 1;
        if (slab >= RING && !mbar_wait(smem_u32(&bars.empty[slot0]), ph0 ^ 1))
          atomicOr(&p.hdr->status, NAJU_ST_MMA_TIMEOUT);
        s_tile[it & 1] = tile;
        if (tile < 0) {  // sentinel: wake the consumers without data
          mbar_arrive(smem_u32(&bars.full[slot0]));
          mbar_arrive(smem_u32(&bars.bc_full[it & 1]));
        } else {
          const int per_chunk = p.B * p.ndt;
          const int c = tile / per_chunk, rem = tile % per_chunk;
          const int b = rem / p.ndt, d0 = (rem % p.ndt) * kDT, t0 = c * Q;
          // raw B and C rows of the chunk (buffer of this tile parity; freed by the builder)
          if (it >= 2 && !mbar_wait(smem_u32(&bars.bc_empty[it & 1]), ((it >> 1) & 1) ^ 1))
            atomicOr(&p.hdr->status, NAJU_ST_MMA_TIMEOUT);
          {
            const uint32_t bar = smem_u32(&bars.bc_full[it & 1]);
            const uint32_t dst = sbase + SM::off_bc + (it & 1) * 2 * BC_BYTES;
            mbar_arrive_expect_tx(bar, 2 * BC_BYTES);
            tma_load_3d(dst, &maps.bm, 0, t0, b, bar);
            tma_load_3d(dst + BC_BYTES, &maps.cm, 0, t0, b, bar);
          }
          for (int k = 0; k < NSLAB; ++k) {
            const uint32_t sidx = slab + k;
            const uint32_t slot = sidx % RING, ph = (sidx / RING) & 1;
            if (k > 0 && sidx >= RING && !mbar_wait(smem_u32(&bars.empty[slot]), ph ^ 1))
              atomicOr(&p.hdr->status, NAJU_ST_MMA_TIMEOUT);
            const uint32_t bar = smem_u32(&bars.full[slot]);
            const uint32_t dst = sbase + SM::off_ring + slot * SM::slab_bytes;
            mbar_arrive_expect_tx(bar, SM::slab_bytes);
            tma_load_3d(dst, &maps.u, d0, t0 + k * SLAB, b, bar);
            tma_load_3d(dst + SLAB * kDT * 2, &maps.fl, d0, t0 + k * SLAB, b, bar);
            tma_load_3d(dst + SLAB * kDT * (2 + sizeof(TG)), &maps.il, d0, t0 + k * SLAB, b, bar);
          }
        }
      }
      slab += NSLAB;
      tile = __shfl_sync(0xffffffffu, tile, 0);
      if (tile < 0) break;
    }
  } else if (warp == 5) {
    // ===================================================================== operand builder
    unsigned char* s_B1 = smem + SM::off_B1;
    unsigned char* s_B2 = smem + SM::off_B2;
    const int g = lane >> 2, t4 = lane & 3;
    for (int it = 0;; ++it) {
      if (!mbar_wait(smem_u32(&bars.bc_full[it & 1]), (it >> 1) & 1))
        atomicOr(&p.hdr->status, NAJU_ST_MMA_TIMEOUT);
      if (s_tile[it & 1] < 0) break;
      // the previous tile's MMAs must be done with B1 / B2
      if (it >= 1 && !mbar_wait(smem_u32(&bars.ops_empty), (it - 1) & 1))
        atomicOr(&p.hdr->status, NAJU_ST_MMA_TIMEOUT);
      const __nv_bfloat16* Braw = reinterpret_cast<const __nv_bfloat16*>(smem + SM::off_bc + (it & 1) * 2 * BC_BYTES);
      const __nv_bfloat16* Craw = Braw + Q * NS;
      // C columns of B1: row t gets its 32 bytes as two 16-byte chunks
      for (int e = lane; e < Q * 2; e += 32) {
        const int t = e >> 1, half = e & 1;
        *reinterpret_cast<uint4*>(s_B1 + op_off16(t, B1_C * 8 + half * 8, SBO_B1)) =
            *reinterpret_cast<const uint4*>(Craw + t * NS + half * 8);
      }
      // B2 = B^T: row n, column s
      for (int e = lane; e < Q * NS; e += 32) {
        const int s = e / NS, n = e % NS;
        *reinterpret_cast<__nv_bfloat16*>(s_B2 + op_off16(n, s, SBO_B2)) = Braw[e];
      }
      // G = tril(C B^T) in two bf16 terms
#pragma unroll 1
      for (int mt = 0; mt < Q / 16; ++mt) {
        const int r0 = 16 * mt + g, r1 = r0 + 8;
        const uint32_t a0 = *reinterpret_cast<const uint32_t*>(Craw + r0 * NS + 2 * t4);
        const uint32_t a1 = *reinterpret_cast<const uint32_t*>(Craw + r1 * NS + 2 * t4);
        const uint32_t a2 = *reinterpret_cast<const uint32_t*>(Craw + r0 * NS + 2 * t4 + 8);
        const uint32_t a3 = *reinterpret_cast<const uint32_t*>(Craw + r1 * NS + 2 * t4 + 8);
#pragma unroll
        for (int nt = 0; nt < Q / 8; ++nt) {
          float c[4] = {0.f, 0.f, 0.f, 0.f};
          if (8 * nt <= 16 * mt + 15) {
            const uint32_t b0 = *reinterpret_cast<const uint32_t*>(Braw + (8 * nt + g) * NS + 2 * t4);
            const uint32_t b1 = *reinterpret_cast<const uint32_t*>(Braw + (8 * nt + g) * NS + 2 * t4 + 8);
            mma_bf16_16x8x16(c, a0, a1, a2, a3, b0, b1);
          }
          const int s0 = 8 * nt + 2 * t4;
          uint32_t hi, lo;
          split_bf16x2(s0 <= r0 ? c[0] : 0.f, s0 + 1 <= r0 ? c[1] : 0.f, hi, lo);
          *reinterpret_cast<uint32_t*>(s_B1 + op_off16(r0, B1_G1 * 8 + s0, SBO_B1)) = hi;
          *reinterpret_cast<uint32_t*>(s_B1 + op_off16(r0, B1_G2 * 8 + s0, SBO_B1)) = lo;
          split_bf16x2(s0 <= r1 ? c[2] : 0.f, s0 + 1 <= r1 ? c[3] : 0.f, hi, lo);
          *reinterpret_cast<uint32_t*>(s_B1 + op_off16(r1, B1_G1 * 8 + s0, SBO_B1)) = hi;
          *reinterpret_cast<uint32_t*>(s_B1 + op_off16(r1, B1_G2 * 8 + s0, SBO_B1)) = lo;
        }
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(&bars.ops_full));
        mbar_arrive(smem_u32(&bars.bc_empty[it & 1]));
      }
    }
  } else {
    // ===================================================================== compute warps
    unsigned char* s_A = smem + SM::off_A;
    unsigned char* a_row = s_A + static_cast<uint32_t>(tid >> 3) * SBO_A + static_cast<uint32_t>(tid & 7) * 16;
    const uint32_t aA = sbase + SM::off_A, aB1 = sbase + SM::off_B1, aB2 = sbase + SM::off_B2;
    const uint32_t trow = tmem + (static_cast<uint32_t>(warp * 32) << 16);
    const uint32_t id16 = umma_idesc(128, NS, 1), id64 = umma_idesc(128, Q, 1);
    uint32_t slab = 0, mph = 0;  // mph: parity of the next tcgen05.commit phase
    PROF_INIT;
    for (int it = 0;; ++it) {
      // ---- tile hand-over: the first slab's barrier also publishes the tile index
      {
        const uint32_t slot = slab % RING, ph = (slab / RING) & 1;
        if (!mbar_wait(smem_u32(&bars.full[slot]), ph)) atomicOr(&p.hdr->status, NAJU_ST_MMA_TIMEOUT);
      }
      const int tile = s_tile[it & 1];
      if (tile < 0) break;
      PROF_MARK(0);
      TileCoord tcd;
      decode_tile<Q>(static_cast<unsigned>(tile), p.B, p.T, p.D, p.nchunks, p.ndt, tid, tcd);
      const int len = tcd.len;

      // ---- gates, running products, scaled inputs -> this thread's A row
      float Pt[Q];
      float R = 1.f, P = 1.f;
#pragma unroll
      for (int k = 0; k < NSLAB; ++k, ++slab) {
        const uint32_t slot = slab % RING, ph = (slab / RING) & 1;
        if (k > 0 && !mbar_wait(smem_u32(&bars.full[slot]), ph)) atomicOr(&p.hdr->status, NAJU_ST_MMA_TIMEOUT);
        const unsigned char* sl = smem + SM::off_ring + slot * SM::slab_bytes;
        const TA* s_u = reinterpret_cast<const TA*>(sl);
        const TG* s_fl = reinterpret_cast<const TG*>(sl + SLAB * kDT * 2);
        const TG* s_il = s_fl + SLAB * kDT;
#pragma unroll
        for (int j8 = 0; j8 < SLAB / 8; ++j8) {
          float wv[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int tl = 8 * j8 + j, t = k * SLAB + tl;
            const float flv = to_f32(s_fl[tl * kDT + tid]);
            const float ilv = fmaxf(to_f32(s_il[tl * kDT + tid]), -30.f);
            const float uv = to_f32(s_u[tl * kDT + tid]);
            float opa = 1.f + fast_ex2(flv * kNegLog2e);   // 1/f
            const float opb = 1.f + fast_ex2(ilv * kNegLog2e);  // 1/i
            if (t >= len) opa = 1.f;                          // ragged last chunk: neutral step
            R *= opa;
            const float r = fast_rcp(R * opb);
            P = opb * r;                                      // 1/R
            wv[j] = uv * (R * r) * R;                         // u * i * R
            Pt[t] = P;
          }
          uint32_t h0, h1, h2, h3, l0, l1, l2, l3;
          split_bf16x2(wv[0], wv[1], h0, l0);
          split_bf16x2(wv[2], wv[3], h1, l1);
          split_bf16x2(wv[4], wv[5], h2, l2);
          split_bf16x2(wv[6], wv[7], h3, l3);
          const int ch = k * (SLAB / 8) + j8;
          *reinterpret_cast<uint4*>(a_row + (A_W1 + ch) * 128) = make_uint4(h0, h1, h2, h3);
          *reinterpret_cast<uint4*>(a_row + (A_W2 + ch) * 128) = make_uint4(l0, l1, l2, l3);
        }
        mbar_arrive(smem_u32(&bars.empty[slot]));
      }
      PROF_MARK(1);
      const bool deep = !(R < kRMax);  // also catches inf / NaN
      fence_async_smem();
      const bool any_deep = bar_or<1, NCOMPUTE>(deep);

      // the shared operands of this tile (built by warp 5 meanwhile)
      if (tid == 0 && !mbar_wait(smem_u32(&bars.ops_full), it & 1)) atomicOr(&p.hdr->status, NAJU_ST_MMA_TIMEOUT);

      PROF_MARK(2);
      if (any_deep) {
        exact_tile_from_global<TA, TG>(p, tcd, tid);
        if (tid == 0) mbar_arrive(smem_u32(&bars.ops_empty));
        bar_sync<1, NCOMPUTE>();
        continue;
      }

      if (tid == 0) {
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {  // D2 = (w1 | w2) . B^T
          const int ach = (ks < 4 ? A_W1 : A_W2) + 2 * (ks & 3);
          umma_bf16(tmem + Q, umma_desc(aA + ach * 128, 128, SBO_A), umma_desc(aB2 + 2 * (ks & 3) * 128, 128, SBO_B2),
                    id16, ks > 0);
        }
        umma_commit(smem_u32(&bars.d2));
#pragma unroll
        for (int ks = 0; ks < 12; ++ks) {  // D1 = w1.g1 + w1.g2 + w2.g1
          const int ach = (ks < 8 ? A_W1 : A_W2) + 2 * (ks & 3);
          const int bch = ((ks >= 4 && ks < 8) ? B1_G2 : B1_G1) + 2 * (ks & 3);
          umma_bf16(tmem, umma_desc(aA + ach * 128, 128, SBO_A), umma_desc(aB1 + bch * 128, 128, SBO_B1), id64,
                    ks > 0);
        }
      }

      PROF_MARK(3);
      // ---- chunk aggregate from D2, carry-in by look-back
      if (!mbar_wait(smem_u32(&bars.d2), mph)) atomicOr(&p.hdr->status, NAJU_ST_MMA_TIMEOUT);
      tc_fence_after();
      float S[NS], h[NS];
      tmem_ld16(trow + Q, S);
#pragma unroll
      for (int n = 0; n < NS; ++n) S[n] *= P;
      float Pin;
      PROF_MARK(4);
      carry_lookback<NS, true>(p, tcd, tid, S, P, h, Pin);
      PROF_MARK(5);

      // ---- carry-in as two bf16 terms into the A row, then D1 += (h1 | h2) . C
      {
        uint32_t hi[8], lo[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) split_bf16x2(h[2 * q], h[2 * q + 1], hi[q], lo[q]);
        *reinterpret_cast<uint4*>(a_row + (A_H1 + 0) * 128) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<uint4*>(a_row + (A_H1 + 1) * 128) = make_uint4(hi[4], hi[5], hi[6], hi[7]);
        *reinterpret_cast<uint4*>(a_row + (A_H2 + 0) * 128) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        *reinterpret_cast<uint4*>(a_row + (A_H2 + 1) * 128) = make_uint4(lo[4], lo[5], lo[6], lo[7]);
      }
      fence_async_smem();
      tc_fence_before();
      bar_sync<1, NCOMPUTE>();
      if (tid == 0) {
        tc_fence_after();
        umma_bf16(tmem, umma_desc(aA + A_H1 * 128, 128, SBO_A), umma_desc(aB1 + B1_C * 128, 128, SBO_B1), id64, 1u);
        umma_bf16(tmem, umma_desc(aA + A_H2 * 128, 128, SBO_A), umma_desc(aB1 + B1_C * 128, 128, SBO_B1), id64, 1u);
        umma_commit(smem_u32(&bars.d1));
      }
      PROF_MARK(6);
      if (!mbar_wait(smem_u32(&bars.d1), mph)) atomicOr(&p.hdr->status, NAJU_ST_MMA_TIMEOUT);
      tc_fence_after();
      if (tid == 0) mbar_arrive(smem_u32(&bars.ops_empty));  // B1 / B2 may be rebuilt

      PROF_MARK(7);
      // ---- epilogue: y_t = P_t D1[d][t] + D_skip u_t, staged in the (now dead) w1 columns of
      // the A operand (row t -> 256 contiguous bytes) and written out with 16-byte stores
      const float Dv = tcd.d_ok ? p.Dskip[tcd.d] : 0.f;
      const TA* gu = reinterpret_cast<const TA*>(p.u) + tcd.b * p.u_sb + static_cast<int64_t>(tcd.t0) * p.u_st + tcd.d;
#pragma unroll
      for (int q = 0; q < Q / 16; ++q) {
        float v[16];
        tmem_ld16(trow + 16 * q, v);
        if (q == 0) PROF_MARK(10);
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          const int t = 16 * q + k;
          float yv = Pt[t] * v[k];
          if (Dv != 0.f && t < len) yv = fmaf(Dv, to_f32(gu[static_cast<int64_t>(t) * p.u_st]), yv);
          *reinterpret_cast<TA*>(s_A + (t >> 3) * SBO_A + A_W1 * 128 + (t & 7) * 256 + tid * 2) = from_f32<TA>(yv);
        }
        if (q == 0) PROF_MARK(11);
      }
      tc_fence_before();
      bar_sync<1, NCOMPUTE>();
      {
        TA* gy = reinterpret_cast<TA*>(p.y) + (static_cast<int64_t>(tcd.b) * p.T + tcd.t0) * p.D + tcd.d0;
#pragma unroll
        for (int i = 0; i < (Q * kDT * 2 / 16) / NCOMPUTE; ++i) {
          const int v16 = i * NCOMPUTE + tid, t = v16 >> 4, c16 = v16 & 15;
          if (t < len && c16 * 8 < tcd.cols) {
            const uint4 val = *reinterpret_cast<const uint4*>(s_A + (t >> 3) * SBO_A + A_W1 * 128 + (t & 7) * 256 + c16 * 16);
            *reinterpret_cast<uint4*>(gy + static_cast<int64_t>(t) * p.D + c16 * 8) = val;
          }
        }
      }
      float xend[NS];
#pragma unroll
      for (int n = 0; n < NS; ++n) xend[n] = fmaf(P, h[n], S[n]);
      write_final<NS>(p, tcd, xend, P * Pin);
      mph ^= 1;
      PROF_MARK(8);
      bar_sync<1, NCOMPUTE>();  // TMEM and the A rows are free for the next tile
      PROF_MARK(9);
    }
  }
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}

}  // namespace tc2

#ifdef NAJU_PROF
}  // namespace naju
extern "C" int naju_b200_debug_prof(unsigned long long* out16, int reset) {
  if (reset) {
    unsigned long long z[16] = {};
    return static_cast<int>(cudaMemcpyToSymbol(naju::tc2::g_prof, z, sizeof(z)));
  }
  return static_cast<int>(cudaMemcpyFromSymbol(out16, naju::tc2::g_prof, 16 * sizeof(unsigned long long)));
}
namespace naju {
#endif

// ------------------------------------------------------------------------------ host side
namespace {

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                             const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(sym);
  }
  return fn;
}

CUtensorMapDataType tm_dtype(int dt) {
  return dt == NAJU_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                        : dt == NAJU_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
}

// [B][T][inner] tensor with element strides (sb, st, 1); box = (box_inner, box_t, 1)
bool make_map(CUtensorMap* m, const void* base, int dt, int64_t B, int64_t T, int64_t inner, int64_t sb,
              int64_t st, int box_inner, int box_t) {
  const int es = dt == NAJU_F32 ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return false;
  if ((st * es) % 16 != 0 || (sb * es) % 16 != 0 || (box_inner * es) % 16 != 0) return false;
  if (B > 1 && sb < st) return false;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(T), static_cast<cuuint64_t>(B)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(st * es), static_cast<cuuint64_t>((B > 1 ? sb : st * T) * es)};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_t), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  return fn(m, tm_dtype(dt), 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

template <typename TA, typename TG>
int launch_tc2_t(const FwdParams& p, const Geometry& g, const tc2::Maps& maps, cudaStream_t st) {
  const size_t smem = tc2::Smem<TG>::total;
  auto kern = tc2::fwd_tc2_kernel<TA, TG>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return static_cast<int>(e);
  const int64_t grid = std::min<int64_t>(g.ntiles, 2LL * sm_count());
  kern<<<static_cast<unsigned>(grid), tc2::NTHREADS, smem, st>>>(p, maps, static_cast<int>(g.ntiles));
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

// Returns -1000 if this problem cannot take the TMA-fed kernel (caller then uses another one).
int launch_fwd_tc2(const FwdParams& p, const Geometry& g, int act, int gate, int bc, void* stream) {
  const bool act16 = act == NAJU_BF16 || act == NAJU_F16;
  if (!(g.N == tc2::NS && g.TC == tc2::Q && act16 && bc == NAJU_BF16 && (gate == act || gate == NAJU_F32)))
    return -1000;
  if (g.ntiles >= (1LL << 31)) return -1000;
  tc2::Maps maps;
  const bool ok =
      make_map(&maps.u, p.u, act, g.B, g.T, g.D, p.u_sb, p.u_st, kDT, tc2::SLAB) &&
      make_map(&maps.fl, p.fl, gate, g.B, g.T, g.D, p.fl_sb, p.fl_st, kDT, tc2::SLAB) &&
      make_map(&maps.il, p.il, gate, g.B, g.T, g.D, p.il_sb, p.il_st, kDT, tc2::SLAB) &&
      make_map(&maps.bm, p.Bm, bc, g.B, g.T, g.N, p.bm_sb, p.bm_st, tc2::NS, tc2::Q) &&
      make_map(&maps.cm, p.Cm, bc, g.B, g.T, g.N, p.cm_sb, p.cm_st, tc2::NS, tc2::Q);
  if (!ok) return -1000;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (act == NAJU_BF16 && gate == NAJU_BF16) return launch_tc2_t<__nv_bfloat16, __nv_bfloat16>(p, g, maps, st);
  if (act == NAJU_BF16 && gate == NAJU_F32) return launch_tc2_t<__nv_bfloat16, float>(p, g, maps, st);
  if (act == NAJU_F16 && gate == NAJU_F16) return launch_tc2_t<__half, __half>(p, g, maps, st);
  if (act == NAJU_F16 && gate == NAJU_F32) return launch_tc2_t<__half, float>(p, g, maps, st);
  return -1000;
}

}  // namespace naju
