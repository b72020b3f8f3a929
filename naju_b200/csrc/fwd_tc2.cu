// Forward gated scan, chunked (state-expansion) form: persistent, TMA-fed, warp-specialised,
// tcgen05/TMEM.
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
// One persistent CTA per SM, eleven warps in five roles, tiles flowing through a two-stage
// pipeline (A rows, shared operands and TMEM accumulators are double buffered):
//   warp 8      TMA producer: takes tile tickets (time-major, so a chunk's predecessor is always
//               already owned by a running CTA) and streams u / f_logit / i_logit in 16-step
//               slabs through a 4-deep mbarrier ring, plus the chunk's B and C rows.
//   warps 4-7   gate warps, thread = channel: sigmoids, running products, the channel's A-operand
//               row (K-major, no swizzle) and P_t, which goes to TMEM with tcgen05.st.
//   warp 9      operand builder: C | g1 | g2 and B^T of the tile with mma.sync.
//   warp 10     MMA issuer: one thread issues every tcgen05.mma and tcgen05.commit.
//   warps 0-3   carry/epilogue warps, thread = channel: chunk aggregate from D2, carry across chunks
//               by the bounded decoupled look-back, carry-in row for the last MMA, then
//               y_t = P_t D1[d][t] read back from TMEM (lane = channel), staged in shared memory and
//               written with 16-byte stores.
// So the latency-bound carry of tile i overlaps the throughput-bound gate work of tile i+1.
// A tile whose retention product falls below 2^-80 in any channel (deep gates) cannot use the
// 1/P_t factorisation; the carry/epilogue warps then run the exact two-pass recurrence for that
// tile straight from global memory.  Every wait (mbarrier, look-back flag) is bounded.
#include <algorithm>
#include <type_traits>

#include "fwd_common.cuh"
#include "tc_common.cuh"
#include "tma_host.h"

namespace naju {
namespace tc2 {

using namespace tcx;

constexpr int Q = 64, NS = 16, SLAB = 16, NSLAB = Q / SLAB, RING = 4, NSTAGE = 2;
constexpr int NGROUP = 128, NTHREADS = 352;
// A operand rows (bf16).  w rows: [w1 64 | w2 64] = 16 chunks of 8 elements (one buffer per
// stage).  h rows: [h1 16 | h2 16] = 4 chunks (single buffer).
constexpr int AW_W1 = 0, AW_W2 = 8;
constexpr uint32_t SBO_AW = 16 * 128, AW_BYTES = 16 * SBO_AW;  // 32768
constexpr int AH_H1 = 0, AH_H2 = 2;
constexpr uint32_t SBO_AH = 4 * 128, AH_BYTES = 16 * SBO_AH;   // 8192
// B1 operand row t (bf16): [C 16 | g1 64 | g2 64] = 18 chunks
constexpr int B1_CH = 18, B1_C = 0, B1_G1 = 2, B1_G2 = 10;
constexpr uint32_t SBO_B1 = B1_CH * 128, B1_BYTES = 8 * SBO_B1;  // 18432
// B2 operand row n (bf16): [B^T 64] = 8 chunks
constexpr uint32_t SBO_B2 = 8 * 128, B2_BYTES = 2 * SBO_B2;  // 2048
constexpr uint32_t BC_BYTES = Q * NS * 2;                      // one raw B (or C) tile, bf16
// TMEM columns of a stage: D1 [0,64), D2 [64,80), P_t [96,160)
constexpr uint32_t TM_D1 = 0, TM_D2 = 64, TM_P = 96, TM_STAGE = 160, TMEM_COLS = 512;
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
    if ((tid & 127) == 0) {                                                    \
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
  static constexpr uint32_t off_AW = off_ring + RING * slab_bytes;  // [NSTAGE]
  static constexpr uint32_t off_AH = off_AW + NSTAGE * AW_BYTES;
  static constexpr uint32_t off_B1 = off_AH + AH_BYTES;             // [NSTAGE]
  static constexpr uint32_t off_B2 = off_B1 + NSTAGE * B1_BYTES;    // [NSTAGE]
  static constexpr uint32_t off_bc = off_B2 + NSTAGE * B2_BYTES;    // [2 tiles][B raw | C raw]
  static constexpr uint32_t total = off_bc + 2 * 2 * BC_BYTES;
};

struct Bars {
  unsigned long long full[RING], empty[RING];   // input slabs (producer -> gate warps)
  unsigned long long bc_full[2], bc_empty[2];   // raw B/C rows per tile parity
  unsigned long long a_full[NSTAGE];            // gate warps -> MMA issuer (A rows + P_t written)
  unsigned long long ops_full[NSTAGE];          // builder -> MMA issuer
  unsigned long long d2_full[NSTAGE];           // D2 (and the first part of D1) issued & complete
  unsigned long long h_ready;                   // carry warps -> MMA issuer (carry-in row written)
  unsigned long long d1_full;                   // D1 complete
  unsigned long long stage_free[NSTAGE];        // carry/epilogue warps -> everyone upstream
};

// Exact two-pass recurrence of one tile straight from global memory (deep-gate tiles only); the
// carry goes through the look-back (hw / Pw are scratch).
template <typename TA, typename TG>
__device__ __noinline__ void exact_tile_from_global(const FwdParams& p, const TileCoord& tc, int tid,
                                                    float (&hw)[NS], float& Pw) {
  const TA* gu = reinterpret_cast<const TA*>(p.u) + tc.b * p.u_sb + static_cast<int64_t>(tc.t0) * p.u_st + tc.d;
  const TG* gf = reinterpret_cast<const TG*>(p.fl) + tc.b * p.fl_sb + static_cast<int64_t>(tc.t0) * p.fl_st + tc.d;
  const TG* gi = reinterpret_cast<const TG*>(p.il) + tc.b * p.il_sb + static_cast<int64_t>(tc.t0) * p.il_st + tc.d;
  const int64_t bbase = tc.b * p.bm_sb + static_cast<int64_t>(tc.t0) * p.bm_st;
  const int64_t cbase = tc.b * p.cm_sb + static_cast<int64_t>(tc.t0) * p.cm_st;
  float x[NS], h[NS];
  float P = 1.f, Pin;
  {
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
  }
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
      h[n] = fmaf(f, h[n], w * bv);
      acc = fmaf(cv, h[n], acc);
    }
    if (tc.d_ok) gy[static_cast<int64_t>(t) * p.D] = from_f32<TA>(fmaf(Dv, ut, acc));
  }
  {
    write_final<NS>(p, tc, h, P * Pin);
  }
}

// Tiles come from the time-major ticket and the carry crosses CTAs by look-back: the form for
// problems with too few channel tiles to fill the GPU by walking them along time (fwd_tc3.cu).
template <typename TA, typename TG>
__global__ void __launch_bounds__(NTHREADS, 1)
fwd_tc2_kernel(const FwdParams p, const __grid_constant__ Maps maps, const int ntiles) {
  using SM = Smem<TG>;
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ Bars bars;
  __shared__ int s_tile[2];                 // producer -> gate warps / builder (by tile parity)
  __shared__ int s_stage_tile[NSTAGE];      // gate warps -> MMA issuer / carry warps
  __shared__ int s_stage_deep[NSTAGE];
  __shared__ unsigned int s_tmem;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t sbase = smem_u32(smem);

  if (tid == 0) {
    for (int i = 0; i < RING; ++i) {
      mbar_init(smem_u32(&bars.full[i]), 1);
      mbar_init(smem_u32(&bars.empty[i]), NGROUP);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars.bc_full[i]), 1);
      mbar_init(smem_u32(&bars.bc_empty[i]), 1);
    }
    for (int i = 0; i < NSTAGE; ++i) {
      mbar_init(smem_u32(&bars.a_full[i]), NGROUP);
      mbar_init(smem_u32(&bars.ops_full[i]), 1);
      mbar_init(smem_u32(&bars.d2_full[i]), 1);
      mbar_init(smem_u32(&bars.stage_free[i]), NGROUP);
    }
    mbar_init(smem_u32(&bars.h_ready), NGROUP);
    mbar_init(smem_u32(&bars.d1_full), 1);
    mbar_init_fence();
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
  // tell the backward that the chunked forward ran (it has watched every tile for deep gates)
  if (blockIdx.x == 0 && tid == 0) {
    atomicOr(p.fwd_form, 1);
    p.hdr->form = NAJU_FORM_TC_TICKET;
  }

  if (warp == 8) {
    // ===================================================================== TMA producer
    uint32_t slab = 0;  // running slab counter across tiles
    for (int it = 0;; ++it) {
      int tile = 0;
      if (lane == 0) {
        {
          const unsigned ticket = atomicAdd(&p.hdr->ticket, 1u);
          tile = ticket < static_cast<unsigned>(ntiles) ? static_cast<int>(ticket) : -1;
        }
        // s_tile[it & 1] was last read for tile it-2; the gate warps have moved past that tile
        // (they released a slab of tile it-1) before the ring lets the producer get this far.
        const uint32_t slot0 = slab % RING, ph0 = (slab / RING) & 1;
        if (slab >= RING && !mbar_wait(smem_u32(&bars.empty[slot0]), ph0 ^ 1)) timeout();
        if (it >= 2 && !mbar_wait(smem_u32(&bars.bc_empty[it & 1]), ((it >> 1) & 1) ^ 1)) timeout();
        s_tile[it & 1] = tile;
        if (tile < 0) {  // sentinel: wake the consumers without data
          mbar_arrive(smem_u32(&bars.full[slot0]));
          mbar_arrive(smem_u32(&bars.bc_full[it & 1]));
        } else {
          const int per_chunk = p.B * p.ndt;
          const int c = tile / per_chunk, rem = tile % per_chunk;
          const int b = rem / p.ndt, d0 = (rem % p.ndt) * kDT, t0 = c * Q;
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
            if (k > 0 && sidx >= RING && !mbar_wait(smem_u32(&bars.empty[slot]), ph ^ 1)) timeout();
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
  } else if (warp == 9) {
    // ===================================================================== operand builder
    const int g = lane >> 2, t4 = lane & 3;
    for (int it = 0;; ++it) {
      const int st = it & 1;
      if (!mbar_wait(smem_u32(&bars.bc_full[st]), (it >> 1) & 1)) timeout();
      if (s_tile[st] < 0) break;
      // stage st: the tile two back must be completely done with B1 / B2
      if (it >= NSTAGE && !mbar_wait(smem_u32(&bars.stage_free[st]), ((it >> 1) & 1) ^ 1)) timeout();
      unsigned char* s_B1 = smem + SM::off_B1 + st * B1_BYTES;
      unsigned char* s_B2 = smem + SM::off_B2 + st * B2_BYTES;
      const __nv_bfloat16* Braw = reinterpret_cast<const __nv_bfloat16*>(smem + SM::off_bc + st * 2 * BC_BYTES);
      const __nv_bfloat16* Craw = Braw + Q * NS;
      // C columns of B1: row t gets its 32 bytes as two 16-byte chunks
      for (int e = lane; e < Q * 2; e += 32) {
        const int t = e >> 1, half = e & 1;
        *reinterpret_cast<uint4*>(s_B1 + op_off16(t, B1_C * 8 + half * 8, SBO_B1)) =
            *reinterpret_cast<const uint4*>(Craw + t * NS + half * 8);
      }
      // B2 = B^T: (row n, eight consecutive columns s) per store
      for (int e = lane; e < NS * (Q / 8); e += 32) {
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
      // G = tril(C B^T) in two bf16 terms (blocks above the diagonal stay zero)
#pragma unroll 1
      for (int mt = 0; mt < Q / 16; ++mt) {
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
        mbar_arrive(smem_u32(&bars.ops_full[st]));
        mbar_arrive(smem_u32(&bars.bc_empty[st]));
      }
    }
  } else if (warp == 10) {
    // ===================================================================== MMA issuer
    const uint32_t id16 = umma_idesc(128, NS, 1), id64 = umma_idesc(128, Q, 1);
    // operand addresses are fixed: build the descriptors once, offset the address field per use
    const uint64_t dAW0 = umma_desc(sbase + SM::off_AW, 128, SBO_AW), dAH = umma_desc(sbase + SM::off_AH, 128, SBO_AH);
    const uint64_t dB10 = umma_desc(sbase + SM::off_B1, 128, SBO_B1), dB20 = umma_desc(sbase + SM::off_B2, 128, SBO_B2);
    auto off = [](uint32_t bytes) { return static_cast<uint64_t>(bytes >> 4); };
    uint32_t hph = 0;  // parity of the next h_ready phase (one per tile)
    for (int it = 0;; ++it) {
      const int st = it & 1;
      const uint32_t par = (it >> 1) & 1;
      int tile = 0, deep = 0;
      if (lane == 0) {
        if (!mbar_wait(smem_u32(&bars.a_full[st]), par)) timeout();
        tile = s_stage_tile[st];
        deep = s_stage_deep[st];
        if (tile < 0) {
          mbar_arrive(smem_u32(&bars.d2_full[st]));  // end marker: pass it on
        } else if (deep) {
          // nothing to compute; pass the stage on and consume this tile's carry-in phase so that
          // the h_ready phases stay aligned with the tile count
          mbar_arrive(smem_u32(&bars.d2_full[st]));
          if (!mbar_wait(smem_u32(&bars.h_ready), hph)) timeout();
        } else {
          if (!mbar_wait(smem_u32(&bars.ops_full[st]), par)) timeout();
          tc_fence_after();
          const uint64_t dAW = dAW0 + off(st * AW_BYTES), dB1 = dB10 + off(st * B1_BYTES), dB2 = dB20 + off(st * B2_BYTES);
          const uint32_t tst = tmem + st * TM_STAGE;
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {  // D2 = (w1 | w2) . B^T
            const int ach = (ks < 4 ? AW_W1 : AW_W2) + 2 * (ks & 3);
            umma_bf16(tst + TM_D2, dAW + off(ach * 128), dB2 + off(2 * (ks & 3) * 128), id16, ks > 0);
          }
          umma_commit(smem_u32(&bars.d2_full[st]));
#ifdef NAJU_PROF
          {
            const long long t_a = clock64();
            mbar_wait(smem_u32(&bars.d2_full[st]), par);
            atomicAdd(&g_prof[12], static_cast<unsigned long long>(clock64() - t_a));
          }
#endif
#pragma unroll
          for (int ks = 0; ks < 12; ++ks) {  // D1 = w1.g1 + w1.g2 + w2.g1
            const int ach = (ks < 8 ? AW_W1 : AW_W2) + 2 * (ks & 3);
            const int bch = ((ks >= 4 && ks < 8) ? B1_G2 : B1_G1) + 2 * (ks & 3);
            umma_bf16(tst + TM_D1, dAW + off(ach * 128), dB1 + off(bch * 128), id64, ks > 0);
          }
#ifdef NAJU_PROF
          const long long t_b = clock64();
#endif
          // D1 += (h1 | h2) . C once the carry warps have resolved the carry-in
          if (!mbar_wait(smem_u32(&bars.h_ready), hph)) timeout();
#ifdef NAJU_PROF
          atomicAdd(&g_prof[13], static_cast<unsigned long long>(clock64() - t_b));
          const long long t_c = clock64();
#endif
          tc_fence_after();
          umma_bf16(tst + TM_D1, dAH + off(AH_H1 * 128), dB1 + off(B1_C * 128), id64, 1u);
          umma_bf16(tst + TM_D1, dAH + off(AH_H2 * 128), dB1 + off(B1_C * 128), id64, 1u);
          umma_commit(smem_u32(&bars.d1_full));
#ifdef NAJU_PROF
          mbar_wait(smem_u32(&bars.d1_full), (unsigned)(it & 1));
          atomicAdd(&g_prof[14], static_cast<unsigned long long>(clock64() - t_c));
#endif
        }
      }
      tile = __shfl_sync(0xffffffffu, tile, 0);
      deep = __shfl_sync(0xffffffffu, deep, 0);
      if (tile < 0) break;
      hph ^= 1;
    }
  } else if (warp >= 4) {
    // ===================================================================== gate warps
    const int q = tid - NGROUP;  // channel within the tile
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    uint32_t slab = 0;
    PROF_INIT;
    for (int it = 0;; ++it) {
      const int st = it & 1;
      {
        const uint32_t slot = slab % RING, ph = (slab / RING) & 1;
        if (!mbar_wait(smem_u32(&bars.full[slot]), ph)) timeout();
      }
      const int tile = s_tile[st];
      if (it >= NSTAGE && !mbar_wait(smem_u32(&bars.stage_free[st]), ((it >> 1) & 1) ^ 1)) timeout();
      if (tile < 0) {
        if (q == 0) s_stage_tile[st] = -1;
        mbar_arrive(smem_u32(&bars.a_full[st]));
        break;
      }
      tc_fence_after();
      PROF_MARK(8);
      const int t0 = (tile / (p.B * p.ndt)) * Q;
      const int len = min(Q, p.T - t0);
      unsigned char* a_row = smem + SM::off_AW + st * AW_BYTES + static_cast<uint32_t>(q >> 3) * SBO_AW +
                             static_cast<uint32_t>(q & 7) * 16;
      const uint32_t tP = tmem + st * TM_STAGE + TM_P + lane_off;
      float R = 1.f, P = 1.f;
#pragma unroll 1
      for (int k = 0; k < NSLAB; ++k, ++slab) {
        const uint32_t slot = slab % RING, ph = (slab / RING) & 1;
        PROF_MARK(9);
        if (k > 0 && !mbar_wait(smem_u32(&bars.full[slot]), ph)) timeout();
        PROF_MARK(11);
        const unsigned char* sl = smem + SM::off_ring + slot * SM::slab_bytes;
        const TA* s_u = reinterpret_cast<const TA*>(sl);
        const TG* s_fl = reinterpret_cast<const TG*>(sl + SLAB * kDT * 2);
        const TG* s_il = s_fl + SLAB * kDT;
#pragma unroll
        for (int j8 = 0; j8 < SLAB / 8; ++j8) {
          float wv[8];
          uint32_t pv[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int tl = 8 * j8 + j;
            const float flv = ld_as_f32(s_fl, tl * kDT + q);
            const float ilv = fmaxf(ld_as_f32(s_il, tl * kDT + q), -30.f);
            const float uv = ld_as_f32(s_u, tl * kDT + q);
            float opa = 1.f + fast_ex2(flv * kNegLog2e);     // 1/f
            const float opb = 1.f + fast_ex2(ilv * kNegLog2e);  // 1/i
            if (k * SLAB + tl >= len) opa = 1.f;              // ragged last chunk: neutral step
            R *= opa;
            const float r = fast_rcp(R * opb);
            P = opb * r;                                      // 1/R
            wv[j] = uv * (R * r) * R;                         // u * i * R
            pv[j] = __float_as_uint(P);
          }
          uint32_t h0, h1, h2, h3, l0, l1, l2, l3;
          split_bf16x2(wv[0], wv[1], h0, l0);
          split_bf16x2(wv[2], wv[3], h1, l1);
          split_bf16x2(wv[4], wv[5], h2, l2);
          split_bf16x2(wv[6], wv[7], h3, l3);
          const int ch = k * (SLAB / 8) + j8;
          *reinterpret_cast<uint4*>(a_row + (AW_W1 + ch) * 128) = make_uint4(h0, h1, h2, h3);
          *reinterpret_cast<uint4*>(a_row + (AW_W2 + ch) * 128) = make_uint4(l0, l1, l2, l3);
#if defined(NAJU_EXP) && (NAJU_EXP & 2)
          if (ch == 7)
#endif
          asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(tP + 8 * ch),
                       "r"(pv[0]), "r"(pv[1]), "r"(pv[2]), "r"(pv[3]), "r"(pv[4]), "r"(pv[5]), "r"(pv[6]), "r"(pv[7])
                       : "memory");
        }
        mbar_arrive(smem_u32(&bars.empty[slot]));
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      PROF_MARK(9);
      const bool deep = !(R < kRMax);  // also catches inf / NaN
      const bool any_deep = bar_or<2, NGROUP>(deep);
      if (q == 0) {
        s_stage_tile[st] = tile;
        s_stage_deep[st] = any_deep ? 1 : 0;
      }
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(smem_u32(&bars.a_full[st]));
      PROF_MARK(10);
    }
  } else {
    // ===================================================================== carry / epilogue warps
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    unsigned char* h_row = smem + SM::off_AH + static_cast<uint32_t>(tid >> 3) * SBO_AH + static_cast<uint32_t>(tid & 7) * 16;
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
    uint32_t dph = 0;  // parity of the next d1_full phase (normal tiles only)
    float hc[NS];  // scratch for the exact path
    float Pc = 1.f;
    // Exactly one carry-in row (one h_ready phase) is posted per tile, deep tiles included.
    PROF_INIT;
    for (int it = 0;; ++it) {
      const int st = it & 1;
      if (!mbar_wait(smem_u32(&bars.d2_full[st]), (it >> 1) & 1)) timeout();
      const int tile = s_stage_tile[st];
      if (tile < 0) break;
      PROF_MARK(0);
      TileCoord tcd;
      decode_tile<Q>(static_cast<unsigned>(tile), p.B, p.T, p.D, p.nchunks, p.ndt, tid, tcd);
      const int len = tcd.len;
      if (s_stage_deep[st]) {
        if (tid == 0) atomicOr(p.fwd_form, 2);
        exact_tile_from_global<TA, TG>(p, tcd, tid, hc, Pc);
        {
          mbar_arrive(smem_u32(&bars.h_ready));  // keep the phase count: one per tile
        }
        mbar_arrive(smem_u32(&bars.stage_free[st]));
        continue;
      }
      const float Dv = tcd.d_ok ? __ldg(p.Dskip + tcd.d) : 0.f;
      tc_fence_after();
      const uint32_t trow = tmem + st * TM_STAGE + lane_off;
      // ---- chunk aggregate from D2 (P_Q is the last P_t)
      float S[NS];
      float P;
      {
        uint32_t sr[16], pl[16];
        tmem_ld16_async(trow + TM_D2, sr);
        tmem_ld16_async(trow + TM_P + 48, pl);
        tmem_ld_wait16(sr);
        tmem_ld_wait16(pl);
        P = __uint_as_float(pl[15]);
#pragma unroll
        for (int n = 0; n < NS; ++n) S[n] = __uint_as_float(sr[n]) * P;
      }
      PROF_MARK(1);
      {
        float h[NS], Pin;
        carry_lookback<NS, true>(p, tcd, tid, S, P, h, Pin);
        write_h_row(h);
        float xend[NS];
#pragma unroll
        for (int n = 0; n < NS; ++n) xend[n] = fmaf(P, h[n], S[n]);
        write_final<NS>(p, tcd, xend, P * Pin);
      }
      PROF_MARK(2);
      if (!mbar_wait(smem_u32(&bars.d1_full), dph)) timeout();
      dph ^= 1;
      tc_fence_after();
      PROF_MARK(3);
      
      PROF_MARK(4);

      // ---- epilogue: y_t = P_t D1[d][t] + D_skip u_t, staged in the (now dead) w1 columns of
      // this stage's A rows (row t -> 256 contiguous bytes) and written out with 16-byte stores
      unsigned char* ystage = smem + SM::off_AW + st * AW_BYTES;
      const TA* gu = reinterpret_cast<const TA*>(p.u) + tcd.b * p.u_sb + static_cast<int64_t>(tcd.t0) * p.u_st + tcd.d;
      {
        // TMEM loads are software-pipelined: the next 16 columns are in flight while the current
        // ones are scaled, rounded and staged
        uint32_t v[2][16], pt[2][16];
        tmem_ld16_async(trow + TM_D1, v[0]);
        tmem_ld16_async(trow + TM_P, pt[0]);
        tmem_ld_wait16(v[0]);
        tmem_ld_wait16(pt[0]);
#pragma unroll
        for (int qq = 0; qq < Q / 16; ++qq) {
          const int cur = qq & 1, nxt = cur ^ 1;
          if (qq + 1 < Q / 16) {
            tmem_ld16_async(trow + TM_D1 + 16 * (qq + 1), v[nxt]);
            tmem_ld16_async(trow + TM_P + 16 * (qq + 1), pt[nxt]);
          }
#pragma unroll
          for (int k = 0; k < 16; k += 2) {
            const int t = 16 * qq + k;
            float y0 = __uint_as_float(pt[cur][k]) * __uint_as_float(v[cur][k]);
            float y1 = __uint_as_float(pt[cur][k + 1]) * __uint_as_float(v[cur][k + 1]);
            if (Dv != 0.f) {
              if (t < len) y0 = fmaf(Dv, to_f32(gu[static_cast<int64_t>(t) * p.u_st]), y0);
              if (t + 1 < len) y1 = fmaf(Dv, to_f32(gu[static_cast<int64_t>(t + 1) * p.u_st]), y1);
            }
            unsigned short o0, o1;
            if constexpr (sizeof(TA) == 2 && !std::is_same<TA, __half>::value) {
              const uint32_t pk = pack_bf16x2(y0, y1);  // one conversion for two steps
              o0 = static_cast<unsigned short>(pk & 0xFFFFu);
              o1 = static_cast<unsigned short>(pk >> 16);
            } else {
              const __half2 pk = __floats2half2_rn(y0, y1);
              o0 = __half_as_ushort(__low2half(pk));
              o1 = __half_as_ushort(__high2half(pk));
            }
            *reinterpret_cast<unsigned short*>(ystage + (t >> 3) * SBO_AW + (t & 7) * 256 + tid * 2) = o0;
            *reinterpret_cast<unsigned short*>(ystage + ((t + 1) >> 3) * SBO_AW + ((t + 1) & 7) * 256 + tid * 2) = o1;
          }
          if (qq + 1 < Q / 16) {
            tmem_ld_wait16(v[nxt]);
            tmem_ld_wait16(pt[nxt]);
          }
        }
      }
      PROF_MARK(5);
      tc_fence_before();
      bar_sync<1, NGROUP>();
      {
        TA* gy = reinterpret_cast<TA*>(p.y) + (static_cast<int64_t>(tcd.b) * p.T + tcd.t0) * p.D + tcd.d0;
#pragma unroll
        for (int i = 0; i < (Q * kDT * 2 / 16) / NGROUP; ++i) {
          const int v16 = i * NGROUP + tid, t = v16 >> 4, c16 = v16 & 15;
          if (t < len && c16 * 8 < tcd.cols) {
            const uint4 val = *reinterpret_cast<const uint4*>(ystage + (t >> 3) * SBO_AW + (t & 7) * 256 + c16 * 16);
            *reinterpret_cast<uint4*>(gy + static_cast<int64_t>(t) * p.D + c16 * 8) = val;
          }
        }
      }
      PROF_MARK(6);
      mbar_arrive(smem_u32(&bars.stage_free[st]));
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

template <typename TA, typename TG>
int launch_tc2_m(const FwdParams& p, const Geometry& g, const tc2::Maps& maps, cudaStream_t st) {
  const size_t smem = tc2::Smem<TG>::total;
  auto kern = tc2::fwd_tc2_kernel<TA, TG>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return static_cast<int>(e);
  // one persistent CTA per SM; in walk mode one CTA per channel tile
  const int64_t grid = std::min<int64_t>(g.ntiles, tmah::sm_count());
  kern<<<static_cast<unsigned>(grid), tc2::NTHREADS, smem, st>>>(p, maps, static_cast<int>(g.ntiles));
  return static_cast<int>(cudaGetLastError());
}

template <typename TA, typename TG>
int launch_tc2_t(const FwdParams& p, const Geometry& g, const tc2::Maps& maps, cudaStream_t st) {
  // Problems with enough channel tiles to walk them along time are taken by the newer kernel
  // (fwd_tc3.cu) before this one is asked; what arrives here spreads over time by ticket.
  return launch_tc2_m<TA, TG>(p, g, maps, st);
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
      tmah::make_map(&maps.u, p.u, act, g.B, g.T, g.D, p.u_sb, p.u_st, kDT, tc2::SLAB) &&
      tmah::make_map(&maps.fl, p.fl, gate, g.B, g.T, g.D, p.fl_sb, p.fl_st, kDT, tc2::SLAB) &&
      tmah::make_map(&maps.il, p.il, gate, g.B, g.T, g.D, p.il_sb, p.il_st, kDT, tc2::SLAB) &&
      tmah::make_map(&maps.bm, p.Bm, bc, g.B, g.T, g.N, p.bm_sb, p.bm_st, tc2::NS, tc2::Q) &&
      tmah::make_map(&maps.cm, p.Cm, bc, g.B, g.T, g.N, p.cm_sb, p.cm_st, tc2::NS, tc2::Q);
  if (!ok) return -1000;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (act == NAJU_BF16 && gate == NAJU_BF16) return launch_tc2_t<__nv_bfloat16, __nv_bfloat16>(p, g, maps, st);
  if (act == NAJU_BF16 && gate == NAJU_F32) return launch_tc2_t<__nv_bfloat16, float>(p, g, maps, st);
  if (act == NAJU_F16 && gate == NAJU_F16) return launch_tc2_t<__half, __half>(p, g, maps, st);
  if (act == NAJU_F16 && gate == NAJU_F32) return launch_tc2_t<__half, float>(p, g, maps, st);
  return -1000;
}

}  // namespace naju
