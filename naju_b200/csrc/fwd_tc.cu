// Forward gated scan, chunked (state-expansion) form on tcgen05 tensor cores.
//
// Within a chunk of Q = 64 steps and per channel d, with P_t = prod_{r<=t} f_r, R_t = 1/P_t and
// wt_s = w_s R_s (w = sigmoid(i_logit) u), the recurrence of naju/scan.py:79-93 unrolls to
//
//   y_t   = P_t [ <C_t, h> + sum_{s<=t} (C_t . B_s) wt_s ] + D_skip u_t
//   x_end = P_Q [ h + sum_s wt_s B_s ]
//
// (the same masked-decay contraction naju/chunk_triton.py:79-144 evaluates with tl.dot on
// 16-step sub-blocks).  For a tile of 128 channels both sums are dense GEMMs whose M dimension
// is the channel:
//
//   D1[128 x 64] = A[128 x (2N+64)] . B1[64 x (2N+64)]^T     A row d = [h_hi | h_lo | wt_0..wt_63]
//                                                             B1 row t = [C_t | C_t | G[t,0..63]]
//   D2[128 x N ] = A[:, 2N:] . B2[N x 64]^T                   B2 row n = B_0..63[n]
//
// with G = tril(C B^T).  Thread = channel: it evaluates the gates and the running products of
// its channel, writes its own operand row (tf32, K-major, no swizzle: 8-row x 16-byte core
// matrices) and reads its own accumulator row back from TMEM (lane = channel).  One elected
// thread issues tcgen05.mma (kind::tf32, M=128, cta_group::1); G comes from four warp-level
// mma.sync tiles.  The carry-in state h is split into two tf32 terms so the state keeps fp32
// accuracy across chunks; the carry itself crosses chunks by the same bounded decoupled
// look-back as the exact kernel, and the checkpoints have the same layout.
//
// The 1/P_t factorisation needs prod f >= 2^-80 over the chunk.  A tile where any channel
// violates that (deep retention gates) takes the exact two-pass recurrent path instead, decided
// per tile on the device, so the kernel is exact for any logit without a host round trip.
#include "fwd_common.cuh"

namespace naju {

namespace tc {

constexpr int Q = 64;                 // steps per tile
constexpr int NS = 16;                // padded state width handled by this kernel
constexpr int KH = 2 * NS;            // h_hi | h_lo columns
constexpr int KT = KH + Q;            // operand K extent (96)
constexpr int CH = KT / 4;            // 16-byte chunks per operand row (24)
constexpr uint32_t LBO = 128;         // bytes between consecutive K chunks (core matrices)
constexpr uint32_t SBO_A = CH * 128;  // bytes between 8-row groups of A and B1
constexpr uint32_t SBO_B2 = (Q / 4) * 128;
constexpr int A_BYTES = 16 * SBO_A;   // 128 rows
constexpr int B1_BYTES = 8 * SBO_A;   // 64 rows
constexpr int B2_BYTES = 2 * SBO_B2;  // 16 rows
constexpr uint32_t TMEM_COLS = 128;   // D1: columns [0,64), D2: [64,80)
constexpr float kRMax = 1.0e24f;      // ~2^80

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// shared-memory matrix descriptor: K-major, no swizzle, descriptor version 1 (sm_100)
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}

// instruction descriptor: D fp32, A and B tf32, both K-major, dense
__device__ __forceinline__ uint32_t umma_idesc(int M, int N) {
  return (1u << 4) | (2u << 7) | (2u << 10) | (static_cast<uint32_t>(N >> 3) << 17) |
         (static_cast<uint32_t>(M >> 4) << 24);
}

__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t mbar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar)
               : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mbar_init(uint32_t mbar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mbar), "r"(count) : "memory");
}

// bounded wait on an mbarrier phase; false if the budget ran out
__device__ __forceinline__ bool mbar_wait(uint32_t mbar, uint32_t parity) {
  for (int it = 0; it < kSpinLimit; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(mbar), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n\t"
      "tcgen05.wait::ld.sync.aligned;\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ float tf32_rna(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

__device__ __forceinline__ void mma_tf32_16x8x8(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// byte offset of element (row, k) in a K-major, no-swizzle operand with SBO `sbo`
__device__ __forceinline__ uint32_t op_off(int row, int k, uint32_t sbo) {
  return static_cast<uint32_t>(row >> 3) * sbo + static_cast<uint32_t>(k >> 2) * LBO +
         static_cast<uint32_t>(row & 7) * 16 + static_cast<uint32_t>(k & 3) * 4;
}

}  // namespace tc

template <typename TA, typename TG>
__global__ void __launch_bounds__(kThreads, 2) fwd_tc_kernel(const FwdParams p) {
  using namespace tc;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  TA* s_u = reinterpret_cast<TA*>(smem_raw);                  // [64][128]; reused for y
  TG* s_fl = reinterpret_cast<TG*>(s_u + Q * kDT);            // [64][128]
  TG* s_il = s_fl + Q * kDT;                                  // [64][128]
  unsigned char* s_A = reinterpret_cast<unsigned char*>(s_il + Q * kDT);  // A operand
  float* s_Bf = reinterpret_cast<float*>(s_A + A_BYTES);      // [64][16] fp32 B
  float* s_Cf = s_Bf + Q * NS;                                // [64][16] fp32 C
  // B operands alias the gate tiles, which are dead once every thread has evaluated its gates
  unsigned char* s_B1 = reinterpret_cast<unsigned char*>(s_fl);
  unsigned char* s_B2 = s_B1 + B1_BYTES;
  __shared__ __align__(8) unsigned long long s_mbar[2];
  __shared__ unsigned int s_tmem;
  __shared__ unsigned int s_ticket;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // TMEM first (may wait for a co-resident CTA to free columns), ticket second, so that a CTA
  // never holds a tile that others wait on while it waits for TMEM.
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    mbar_init(smem_u32(&s_mbar[0]), 1);
    mbar_init(smem_u32(&s_mbar[1]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    s_ticket = atomicAdd(&p.hdr->ticket, 1u);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;
  TileCoord tcd;
  const bool tile_ok = decode_tile<Q>(s_ticket, p.B, p.T, p.D, p.nchunks, p.ndt, tid, tcd);
  if (!tile_ok && tid == 0) atomicOr(&p.hdr->status, NAJU_ST_BAD_TILE);  // never expected

  if (tile_ok) {
    const int b = tcd.b, t0 = tcd.t0, len = tcd.len, d0 = tcd.d0, cols = tcd.cols;

    // ---- stage the tile
    load_tile_async(s_u, reinterpret_cast<const TA*>(p.u) + b * p.u_sb + t0 * p.u_st + d0, p.u_st,
                    len, cols, tid);
    load_tile_async(s_fl, reinterpret_cast<const TG*>(p.fl) + b * p.fl_sb + t0 * p.fl_st + d0,
                    p.fl_st, len, cols, tid);
    load_tile_async(s_il, reinterpret_cast<const TG*>(p.il) + b * p.il_sb + t0 * p.il_st + d0,
                    p.il_st, len, cols, tid);
    cp_async_commit();
    for (int e = tid; e < Q * NS; e += kThreads) {
      const int r = e / NS, n = e % NS;
      const bool ok = r < len && n < p.N;
      s_Bf[e] = ok ? load_dyn(p.Bm, p.bc_dtype, b * p.bm_sb + (t0 + r) * p.bm_st + n) : 0.f;
      s_Cf[e] = ok ? load_dyn(p.Cm, p.bc_dtype, b * p.cm_sb + (t0 + r) * p.cm_st + n) : 0.f;
    }
    cp_async_wait_all();
    __syncthreads();

    // ---- gates, running products, scaled inputs -> this thread's A row
    unsigned char* a_row = s_A + static_cast<uint32_t>(tid >> 3) * SBO_A + static_cast<uint32_t>(tid & 7) * 16;
    float Pt[Q];
    float R = 1.f, P = 1.f;
#pragma unroll
    for (int t4 = 0; t4 < Q / 4; ++t4) {
      float wt[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int t = 4 * t4 + k;
        float wv = 0.f;
        if (t < len) {
          const float flv = fmaxf(to_f32(s_fl[t * kDT + tid]), -80.f);
          const float opa = 1.f + __expf(-flv);  // 1/f
          const float f = __fdividef(1.f, opa);
          const float iv = sigmoid_f(to_f32(s_il[t * kDT + tid]));
          R *= opa;
          P *= f;
          wv = iv * to_f32(s_u[t * kDT + tid]) * R;
        }
        Pt[t] = P;
        wt[k] = tf32_rna(wv);
      }
      *reinterpret_cast<float4*>(a_row + (KH / 4 + t4) * LBO) = make_float4(wt[0], wt[1], wt[2], wt[3]);
    }
    const bool deep = !(R < kRMax);  // also catches inf/NaN
    const int any_deep = __syncthreads_or(deep ? 1 : 0);
    const float Dv = tcd.d_ok ? p.Dskip[tcd.d] : 0.f;

    if (any_deep) {
      // exact two-pass recurrent path for this tile
      float x[NS], h[NS];
      float P1, Pin;
      tile_pass1<TA, TG, NS>(s_u, s_fl, s_il, s_Bf, len, tid, x, P1);
      carry_lookback<NS>(p, tcd, tid, x, P1, h, Pin);
      tile_pass2<TA, TG, NS>(s_u, s_fl, s_il, s_Bf, s_Cf, len, tid, Dv, h);
      write_final<NS>(p, tcd, h, P1 * Pin);
    } else {
      // ---- shared operands: B1 = [C | C | tril(C B^T)], B2 = B^T   (gate tiles are dead now)
      for (int e = tid; e < Q * NS; e += kThreads) {
        const int r = e / NS, n = e % NS;
        const float cv = s_Cf[e];
        *reinterpret_cast<float*>(s_B1 + op_off(r, n, SBO_A)) = cv;
        *reinterpret_cast<float*>(s_B1 + op_off(r, NS + n, SBO_A)) = cv;
        *reinterpret_cast<float*>(s_B2 + op_off(n, r, SBO_B2)) = s_Bf[e];
      }
      {
        const int g = lane >> 2, t4 = lane & 3;
        const int r0 = 16 * warp + g, r1 = r0 + 8;
        uint32_t afr[2][4];
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
          afr[ks][0] = __float_as_uint(s_Cf[r0 * NS + 8 * ks + t4]);
          afr[ks][1] = __float_as_uint(s_Cf[r1 * NS + 8 * ks + t4]);
          afr[ks][2] = __float_as_uint(s_Cf[r0 * NS + 8 * ks + t4 + 4]);
          afr[ks][3] = __float_as_uint(s_Cf[r1 * NS + 8 * ks + t4 + 4]);
        }
#pragma unroll
        for (int nt = 0; nt < Q / 8; ++nt) {
          float c[4] = {0.f, 0.f, 0.f, 0.f};
          if (8 * nt <= 16 * warp + 15) {  // tile touches the causal triangle (warp-uniform)
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
              const uint32_t b0 = __float_as_uint(s_Bf[(8 * nt + g) * NS + 8 * ks + t4]);
              const uint32_t b1 = __float_as_uint(s_Bf[(8 * nt + g) * NS + 8 * ks + t4 + 4]);
              mma_tf32_16x8x8(c, afr[ks][0], afr[ks][1], afr[ks][2], afr[ks][3], b0, b1);
            }
          }
          const int s0 = 8 * nt + 2 * t4;
          const float2 v0 = make_float2(s0 <= r0 ? tf32_rna(c[0]) : 0.f, s0 + 1 <= r0 ? tf32_rna(c[1]) : 0.f);
          const float2 v1 = make_float2(s0 <= r1 ? tf32_rna(c[2]) : 0.f, s0 + 1 <= r1 ? tf32_rna(c[3]) : 0.f);
          *reinterpret_cast<float2*>(s_B1 + op_off(r0, KH + s0, SBO_A)) = v0;
          *reinterpret_cast<float2*>(s_B1 + op_off(r1, KH + s0, SBO_A)) = v1;
        }
      }
      fence_async_smem();
      tc_fence_before();
      __syncthreads();

      const uint32_t aA = smem_u32(s_A), aB1 = smem_u32(s_B1), aB2 = smem_u32(s_B2);
      if (tid == 0) {
        tc_fence_after();
        const uint32_t id2 = umma_idesc(128, NS), id1 = umma_idesc(128, Q);
#pragma unroll
        for (int ks = 0; ks < Q / 8; ++ks)  // D2 = wt . B^T
          umma_tf32(tmem + Q, umma_desc(aA + (KH / 4 + 2 * ks) * LBO, LBO, SBO_A),
                    umma_desc(aB2 + 2 * ks * LBO, LBO, SBO_B2), id2, ks > 0);
        umma_commit(smem_u32(&s_mbar[0]));
#pragma unroll
        for (int ks = 0; ks < Q / 8; ++ks)  // D1 = wt . tril(C B^T)^T
          umma_tf32(tmem, umma_desc(aA + (KH / 4 + 2 * ks) * LBO, LBO, SBO_A),
                    umma_desc(aB1 + (KH / 4 + 2 * ks) * LBO, LBO, SBO_A), id1, ks > 0);
      }

      // ---- chunk aggregate from D2, carry-in by look-back
      if (!mbar_wait(smem_u32(&s_mbar[0]), 0)) atomicOr(&p.hdr->status, NAJU_ST_MMA_TIMEOUT);
      tc_fence_after();
      const uint32_t trow = tmem + (static_cast<uint32_t>(warp * 32) << 16);
      float S[NS], h[NS];
      tmem_ld16(trow + Q, S);
#pragma unroll
      for (int n = 0; n < NS; ++n) S[n] *= P;
      float Pin;
      carry_lookback<NS>(p, tcd, tid, S, P, h, Pin);

      // ---- carry-in as two tf32 terms into the A row, then D1 += [h_hi|h_lo] . [C|C]^T
#pragma unroll
      for (int q = 0; q < NS / 4; ++q) {
        float hi[4], lo[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          hi[k] = tf32_rna(h[4 * q + k]);
          lo[k] = tf32_rna(h[4 * q + k] - hi[k]);
        }
        *reinterpret_cast<float4*>(a_row + q * LBO) = make_float4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<float4*>(a_row + (NS / 4 + q) * LBO) = make_float4(lo[0], lo[1], lo[2], lo[3]);
      }
      fence_async_smem();
      tc_fence_before();
      __syncthreads();
      if (tid == 0) {
        tc_fence_after();
        const uint32_t id1 = umma_idesc(128, Q);
#pragma unroll
        for (int ks = 0; ks < KH / 8; ++ks)
          umma_tf32(tmem, umma_desc(aA + 2 * ks * LBO, LBO, SBO_A), umma_desc(aB1 + 2 * ks * LBO, LBO, SBO_A),
                    id1, 1u);
        umma_commit(smem_u32(&s_mbar[1]));
      }
      if (!mbar_wait(smem_u32(&s_mbar[1]), 0)) atomicOr(&p.hdr->status, NAJU_ST_MMA_TIMEOUT);
      tc_fence_after();

      // ---- epilogue: y_t = P_t D1[d][t] + D_skip u_t
#pragma unroll
      for (int q = 0; q < Q / 16; ++q) {
        float v[16];
        tmem_ld16(trow + 16 * q, v);
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          const int t = 16 * q + k;
          if (t < len) {
            const float ut = to_f32(s_u[t * kDT + tid]);
            s_u[t * kDT + tid] = from_f32<TA>(fmaf(Pt[t], v[k], Dv * ut));
          }
        }
      }
      // chunk-end state and total decay of the last chunk
      float xend[NS];
#pragma unroll
      for (int n = 0; n < NS; ++n) xend[n] = fmaf(P, h[n], S[n]);
      write_final<NS>(p, tcd, xend, P * Pin);
    }
    tc_fence_before();
    __syncthreads();
    store_tile(reinterpret_cast<TA*>(p.y) + (static_cast<int64_t>(b) * p.T + t0) * p.D + d0, s_u,
               static_cast<int64_t>(p.D), len, cols, tid);
  }
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tc::TMEM_COLS) : "memory");
  }
}

template <typename TA, typename TG>
static int launch_tc(const FwdParams& p, const Geometry& g, cudaStream_t st) {
  const size_t smem = static_cast<size_t>(tc::Q) * kDT * (sizeof(TA) + 2 * sizeof(TG)) + tc::A_BYTES +
                      2 * static_cast<size_t>(tc::Q) * tc::NS * 4;
  auto kern = fwd_tc_kernel<TA, TG>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem));
  if (e != cudaSuccess) return static_cast<int>(e);
  kern<<<static_cast<unsigned>(g.ntiles), kThreads, smem, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}

bool fwd_tc_supported(const Geometry& g, int act, int gate, int bc) {
  const bool act16 = act == NAJU_BF16 || act == NAJU_F16;
  const bool bc16 = bc == NAJU_BF16 || bc == NAJU_F16;  // exact in tf32
  return g.NS == tc::NS && g.TC == tc::Q && act16 && bc16 && (gate == act || gate == NAJU_F32);
}

int launch_fwd_tc(const FwdParams& p, const Geometry& g, int act, int gate, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (act == NAJU_BF16 && gate == NAJU_BF16) return launch_tc<__nv_bfloat16, __nv_bfloat16>(p, g, st);
  if (act == NAJU_BF16 && gate == NAJU_F32) return launch_tc<__nv_bfloat16, float>(p, g, st);
  if (act == NAJU_F16 && gate == NAJU_F16) return launch_tc<__half, __half>(p, g, st);
  if (act == NAJU_F16 && gate == NAJU_F32) return launch_tc<__half, float>(p, g, st);
  return NAJU_E_DTYPE;
}

}  // namespace naju
