// Single-token recurrent state update for decode: one iteration of the scan recurrence
// (naju/scan.py:87-91 of the reference project, which has no decode entry point).
//
//   state[b,d,n] <- f state[b,d,n] + (i u) B[b,n];   y[b,d] = sum_n C[b,n] state[b,d,n] + D_skip u
//
// Pure HBM streaming of the fp32 state (read once, written once).  Each thread owns four
// consecutive states (one 16-byte load/store); the N/4 lanes that share a channel are
// adjacent, so a warp touches one contiguous 512-byte span per access and the readout is a
// short shuffle reduction.
#include "common.cuh"
#include "params.h"

namespace naju {

constexpr int kStepBlock = 128;  // (measured: 128 threads 20.2 us per launch, 256: 20.8, 512: 22.2)

template <typename TA, typename TG>
__global__ void __launch_bounds__(kStepBlock) step_kernel(float* __restrict__ state, const TA* __restrict__ u,
                                                   const TG* __restrict__ fl, const TG* __restrict__ il,
                                                   const void* __restrict__ Bm, const void* __restrict__ Cm,
                                                   const float* __restrict__ Dskip, TA* __restrict__ y,
                                                   int B, int D, int N, int lpc /* lanes per channel, pow2 */,
                                                   int bc_dtype, int64_t u_sb, int64_t fl_sb, int64_t il_sb,
                                                   int64_t bm_sb, int64_t cm_sb) {
  const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t chan = gid / lpc;           // flat (b, d)
  const int q = static_cast<int>(gid % lpc);  // which group of four states
  const bool ok = chan < static_cast<int64_t>(B) * D;
  float part = 0.f;
  float ut = 0.f;
  int b = 0, d = 0;
  if (ok) {
    b = static_cast<int>(chan / D);
    d = static_cast<int>(chan % D);
    ut = to_f32(u[b * u_sb + d]);
    const float f = sigmoid_f(to_f32(fl[b * fl_sb + d]));
    const float w = sigmoid_f(to_f32(il[b * il_sb + d])) * ut;
    const int n0 = 4 * q;
    float* sp = state + chan * N + n0;
    if (n0 + 4 <= N && (N & 3) == 0) {
      // the state is touched once per token: streaming (evict-first) accesses keep it from pushing
      // the token's small inputs out of L2
      float4 s = __ldcs(reinterpret_cast<const float4*>(sp));
      s.x = fmaf(f, s.x, w * load_dyn(Bm, bc_dtype, b * bm_sb + n0 + 0));
      s.y = fmaf(f, s.y, w * load_dyn(Bm, bc_dtype, b * bm_sb + n0 + 1));
      s.z = fmaf(f, s.z, w * load_dyn(Bm, bc_dtype, b * bm_sb + n0 + 2));
      s.w = fmaf(f, s.w, w * load_dyn(Bm, bc_dtype, b * bm_sb + n0 + 3));
      __stcs(reinterpret_cast<float4*>(sp), s);
      part = s.x * load_dyn(Cm, bc_dtype, b * cm_sb + n0 + 0);
      part = fmaf(s.y, load_dyn(Cm, bc_dtype, b * cm_sb + n0 + 1), part);
      part = fmaf(s.z, load_dyn(Cm, bc_dtype, b * cm_sb + n0 + 2), part);
      part = fmaf(s.w, load_dyn(Cm, bc_dtype, b * cm_sb + n0 + 3), part);
    } else {
      for (int n = n0; n < min(n0 + 4, N); ++n) {
        const float s = fmaf(f, sp[n - n0], w * load_dyn(Bm, bc_dtype, b * bm_sb + n));
        sp[n - n0] = s;
        part = fmaf(s, load_dyn(Cm, bc_dtype, b * cm_sb + n), part);
      }
    }
  }
  // lanes sharing a channel are adjacent and lpc divides 32
  for (int m = lpc >> 1; m >= 1; m >>= 1) part += __shfl_xor_sync(0xffffffffu, part, m);
  if (ok && q == 0) y[static_cast<int64_t>(b) * D + d] = from_f32<TA>(fmaf(Dskip[d], ut, part));
}

template <typename TA, typename TG>
static int launch_t(const naju_scan_desc& d, float* state, const void* u, const void* fl,
                    const void* il, const void* Bm, const void* Cm, const float* Dskip, void* y,
                    cudaStream_t st) {
  int lpc = 1;
  while (lpc * 4 < d.N) lpc <<= 1;  // 1..32
  const int64_t threads = static_cast<int64_t>(d.B) * d.D * lpc;
  const unsigned blocks = static_cast<unsigned>((threads + kStepBlock - 1) / kStepBlock);
  step_kernel<TA, TG><<<blocks, kStepBlock, 0, st>>>(
      state, static_cast<const TA*>(u), static_cast<const TG*>(fl), static_cast<const TG*>(il), Bm,
      Cm, Dskip, static_cast<TA*>(y), d.B, d.D, d.N, lpc, d.bc_dtype, d.u_sb, d.fl_sb, d.il_sb,
      d.bm_sb, d.cm_sb);
  return static_cast<int>(cudaGetLastError());
}

int launch_step(const naju_scan_desc& d, float* state, const void* u, const void* fl, const void* il,
                const void* Bm, const void* Cm, const float* Dskip, void* y, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int a = d.act_dtype, g = d.gate_dtype;
  if (a == NAJU_F32 && g == NAJU_F32) return launch_t<float, float>(d, state, u, fl, il, Bm, Cm, Dskip, y, st);
  if (a == NAJU_BF16 && g == NAJU_BF16) return launch_t<__nv_bfloat16, __nv_bfloat16>(d, state, u, fl, il, Bm, Cm, Dskip, y, st);
  if (a == NAJU_BF16 && g == NAJU_F32) return launch_t<__nv_bfloat16, float>(d, state, u, fl, il, Bm, Cm, Dskip, y, st);
  if (a == NAJU_F16 && g == NAJU_F16) return launch_t<__half, __half>(d, state, u, fl, il, Bm, Cm, Dskip, y, st);
  if (a == NAJU_F16 && g == NAJU_F32) return launch_t<__half, float>(d, state, u, fl, il, Bm, Cm, Dskip, y, st);
  return NAJU_E_DTYPE;
}

}  // namespace naju
