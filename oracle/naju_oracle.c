/* TEST INFRASTRUCTURE — CPU restatement of the Naju gated diagonal scan.
 *
 * This file is the parity oracle for the CUDA path.  It is never linked into,
 * imported by or called from the product library; only the tests, the smoke
 * check and the CPU-baseline leg of the benchmark may use it.
 *
 * Algorithm restated (reference project paths):
 *   forward   naju/scan.py:79-93 (naju_scan_reference):
 *               f = sigmoid(f_logit), i = sigmoid(i_logit)
 *               x_t[n] = f_t x_{t-1}[n] + i_t B_t[n] u_t ,  x_{-1} = h0 (reference: zeros)
 *               y_t    = sum_n C_t[n] x_t[n] + D_skip u_t
 *   backward  the adjoint of that loop, as written out in
 *             naju/cuda/naju_cuda.cu:85-144 (naju_bwd_kernel):
 *               xbar_t = dy_t C_t + f_{t+1} xbar_{t+1}        (terminal: dhT or 0)
 *               dC_t[n] = sum_d dy_t x_t[n]
 *               dB_t[n] = sum_d xbar_t[n] i_t u_t
 *               g_t = sum_n xbar_t[n] B_t[n]
 *               du_t = i_t g_t + D_skip dy_t
 *               d i_logit_t = g_t u_t i_t (1-i_t)
 *               d f_logit_t = <xbar_t, x_{t-1}> f_t (1-f_t)
 *               dD_skip = sum_{b,t} dy_t u_t ,  dh0 = f_0 xbar_0
 *   step      one iteration of naju/scan.py:87-91 from a given state.
 *
 * The initial state h0, the returned final state hT and their adjoints
 * (dhT in, dh0 out) are extensions: the reference always starts from zeros and
 * returns only y.  With h0 = NULL / hT = NULL the functions reduce exactly to
 * the reference.
 *
 * Two arithmetic flavours are exported: *_f32 computes in float exactly like
 * the reference's fp32 path (same operation order per element), *_f64 computes
 * in double from the same float inputs and rounds the results to float once.
 * All arrays are dense row-major float: u,fl,il,y,dy,du,dfl,dil [B,T,D];
 * Bm,Cm,dB,dC [B,T,N]; Dskip,dD [D]; h0,hT,dhT,dh0 [B,D,N].
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define IDX3(b, t, d, T, D) (((size_t)(b) * (T) + (t)) * (D) + (d))

int naju_oracle_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

static inline int naju_oracle_tid(void) {
#ifdef _OPENMP
  return omp_get_thread_num();
#else
  return 0;
#endif
}

#define DEFINE_ORACLE(SUFFIX, real, EXPF)                                                  \
  static inline real sig_##SUFFIX(real x) { return (real)1 / ((real)1 + EXPF(-x)); }       \
                                                                                           \
  void naju_oracle_fwd_##SUFFIX(const float* u, const float* fl, const float* il,          \
                                const float* Bm, const float* Cm, const float* Dskip,      \
                                const float* h0, float* y, float* hT, int B, int T,        \
                                int D, int N) {                                            \
    _Pragma("omp parallel for collapse(2) schedule(static)")                               \
    for (int b = 0; b < B; ++b)                                                            \
      for (int d = 0; d < D; ++d) {                                                        \
        real x[128];                                                                       \
        for (int n = 0; n < N; ++n)                                                        \
          x[n] = h0 ? (real)h0[((size_t)b * D + d) * N + n] : (real)0;                     \
        const real Dv = (real)Dskip[d];                                                    \
        for (int t = 0; t < T; ++t) {                                                      \
          const size_t k = IDX3(b, t, d, T, D);                                            \
          const real f = sig_##SUFFIX((real)fl[k]);                                        \
          const real i = sig_##SUFFIX((real)il[k]);                                        \
          const real ut = (real)u[k];                                                      \
          const float* Bt = Bm + ((size_t)b * T + t) * N;                                  \
          const float* Ct = Cm + ((size_t)b * T + t) * N;                                  \
          real acc = 0;                                                                    \
          for (int n = 0; n < N; ++n) {                                                    \
            x[n] = f * x[n] + i * (real)Bt[n] * ut;                                        \
            acc += (real)Ct[n] * x[n];                                                     \
          }                                                                                \
          y[k] = (float)(acc + Dv * ut);                                                   \
        }                                                                                  \
        if (hT)                                                                            \
          for (int n = 0; n < N; ++n) hT[((size_t)b * D + d) * N + n] = (float)x[n];       \
      }                                                                                    \
  }                                                                                        \
                                                                                           \
  /* returns 0, or -1 when scratch memory could not be allocated */                        \
  int naju_oracle_bwd_##SUFFIX(const float* u, const float* fl, const float* il,           \
                               const float* Bm, const float* Cm, const float* Dskip,       \
                               const float* h0, const float* dy, const float* dhT,         \
                               float* du, float* dfl, float* dil, float* dB, float* dC,    \
                               float* dD, float* dh0, int B, int T, int D, int N) {        \
    int nthreads = naju_oracle_threads();                                                  \
    const size_t tn = (size_t)T * N;                                                       \
    real* accB = (real*)calloc((size_t)nthreads * tn, sizeof(real));                       \
    real* accC = (real*)calloc((size_t)nthreads * tn, sizeof(real));                       \
    real* hist = (real*)malloc((size_t)nthreads * (tn + N) * sizeof(real));                \
    real* accD = (real*)calloc((size_t)D, sizeof(real));                                   \
    if (!accB || !accC || !hist || !accD) {                                                \
      free(accB); free(accC); free(hist); free(accD);                                      \
      return -1;                                                                           \
    }                                                                                      \
    for (int b = 0; b < B; ++b) {                                                          \
      memset(accB, 0, (size_t)nthreads * tn * sizeof(real));                               \
      memset(accC, 0, (size_t)nthreads * tn * sizeof(real));                               \
      _Pragma("omp parallel for schedule(static)")                                         \
      for (int d = 0; d < D; ++d) {                                                        \
        const int tid = naju_oracle_tid();                                                 \
        real* xs = hist + (size_t)tid * (tn + N); /* xs[(t+1)*N+n] = x_t, xs[n] = h0 */    \
        real* aB = accB + (size_t)tid * tn;                                                \
        real* aC = accC + (size_t)tid * tn;                                                \
        for (int n = 0; n < N; ++n)                                                        \
          xs[n] = h0 ? (real)h0[((size_t)b * D + d) * N + n] : (real)0;                    \
        for (int t = 0; t < T; ++t) {                                                      \
          const size_t k = IDX3(b, t, d, T, D);                                            \
          const real f = sig_##SUFFIX((real)fl[k]);                                        \
          const real i = sig_##SUFFIX((real)il[k]);                                        \
          const real ut = (real)u[k];                                                      \
          const float* Bt = Bm + ((size_t)b * T + t) * N;                                  \
          for (int n = 0; n < N; ++n)                                                      \
            xs[(size_t)(t + 1) * N + n] = f * xs[(size_t)t * N + n] + i * (real)Bt[n] * ut;\
        }                                                                                  \
        real carry[128];                                                                   \
        for (int n = 0; n < N; ++n)                                                        \
          carry[n] = dhT ? (real)dhT[((size_t)b * D + d) * N + n] : (real)0;               \
        const real Dv = (real)Dskip[d];                                                    \
        real dDsum = 0;                                                                    \
        for (int t = T - 1; t >= 0; --t) {                                                 \
          const size_t k = IDX3(b, t, d, T, D);                                            \
          const real f = sig_##SUFFIX((real)fl[k]);                                        \
          const real i = sig_##SUFFIX((real)il[k]);                                        \
          const real ut = (real)u[k];                                                      \
          const real dyt = (real)dy[k];                                                    \
          const float* Bt = Bm + ((size_t)b * T + t) * N;                                  \
          const float* Ct = Cm + ((size_t)b * T + t) * N;                                  \
          real dfsum = 0, g = 0;                                                           \
          for (int n = 0; n < N; ++n) {                                                    \
            const real dx = (real)Ct[n] * dyt + carry[n];                                  \
            aC[(size_t)t * N + n] += dyt * xs[(size_t)(t + 1) * N + n];                    \
            aB[(size_t)t * N + n] += dx * i * ut;                                          \
            dfsum += dx * xs[(size_t)t * N + n];                                           \
            g += dx * (real)Bt[n];                                                         \
            carry[n] = f * dx;                                                             \
          }                                                                                \
          dDsum += dyt * ut;                                                               \
          dfl[k] = (float)(dfsum * f * ((real)1 - f));                                     \
          dil[k] = (float)(g * ut * i * ((real)1 - i));                                    \
          du[k] = (float)(dyt * Dv + i * g);                                               \
        }                                                                                  \
        if (dh0)                                                                           \
          for (int n = 0; n < N; ++n) dh0[((size_t)b * D + d) * N + n] = (float)carry[n];  \
        accD[d] += dDsum;                                                                  \
      }                                                                                    \
      for (size_t k = 0; k < tn; ++k) {                                                    \
        real sB = 0, sC = 0;                                                               \
        for (int th = 0; th < nthreads; ++th) {                                            \
          sB += accB[(size_t)th * tn + k];                                                 \
          sC += accC[(size_t)th * tn + k];                                                 \
        }                                                                                  \
        dB[(size_t)b * tn + k] = (float)sB;                                                \
        dC[(size_t)b * tn + k] = (float)sC;                                                \
      }                                                                                    \
    }                                                                                      \
    for (int d = 0; d < D; ++d) dD[d] = (float)accD[d];                                    \
    free(accB); free(accC); free(hist); free(accD);                                        \
    return 0;                                                                              \
  }                                                                                        \
                                                                                           \
  /* one decode step: state [B,D,N] updated in place; u,fl,il,y [B,D]; Bm,Cm [B,N] */      \
  void naju_oracle_step_##SUFFIX(float* state, const float* u, const float* fl,            \
                                 const float* il, const float* Bm, const float* Cm,        \
                                 const float* Dskip, float* y, int B, int D, int N) {      \
    _Pragma("omp parallel for collapse(2) schedule(static)")                               \
    for (int b = 0; b < B; ++b)                                                            \
      for (int d = 0; d < D; ++d) {                                                        \
        const size_t k = (size_t)b * D + d;                                                \
        const real f = sig_##SUFFIX((real)fl[k]);                                          \
        const real i = sig_##SUFFIX((real)il[k]);                                          \
        const real ut = (real)u[k];                                                        \
        real acc = 0;                                                                      \
        for (int n = 0; n < N; ++n) {                                                      \
          const real x = f * (real)state[k * N + n] + i * (real)Bm[(size_t)b * N + n] * ut;\
          state[k * N + n] = (float)x;                                                     \
          acc += (real)Cm[(size_t)b * N + n] * x;                                          \
        }                                                                                  \
        y[k] = (float)(acc + (real)Dskip[d] * ut);                                         \
      }                                                                                    \
  }

DEFINE_ORACLE(f32, float, expf)
DEFINE_ORACLE(f64, double, exp)
