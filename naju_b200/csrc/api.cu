// extern "C" entry points of libnaju_b200.so: argument validation, workspace carving and
// kernel dispatch.  No allocation, no host synchronisation except naju_b200_read_status().
#include <cuda_runtime.h>

#include "naju_b200.h"
#include "params.h"

using namespace naju;

namespace {

size_t dtype_size(int dt) { return dt == NAJU_F32 ? 4 : 2; }

bool dtype_ok(int dt) { return dt == NAJU_F32 || dt == NAJU_BF16 || dt == NAJU_F16; }

bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

int check_desc(const naju_scan_desc* d, bool need_T) {
  if (d == nullptr) return NAJU_E_NULL;
  if (d->B < 0 || d->D < 0 || d->N < 1 || d->N > 128 || (need_T && d->T < 0)) return NAJU_E_SHAPE;
  if (!dtype_ok(d->act_dtype) || !dtype_ok(d->gate_dtype) || !dtype_ok(d->bc_dtype)) return NAJU_E_DTYPE;
  if (!(d->gate_dtype == d->act_dtype || d->gate_dtype == NAJU_F32)) return NAJU_E_DTYPE;
  if ((d->flags & ~(NAJU_FLAG_RECURRENT_ONLY | NAJU_FLAG_CHUNKED_ONLY | NAJU_FLAG_INJECT_TIMEOUT)) != 0)
    return NAJU_E_SHAPE;
  if ((d->flags & NAJU_FLAG_RECURRENT_ONLY) && (d->flags & NAJU_FLAG_CHUNKED_ONLY)) return NAJU_E_SHAPE;
  return NAJU_OK;
}

int check_strides(const naju_scan_desc* d) {
  if (d->u_sd > 1) {  // time-contiguous u: channels u_sd apart, steps adjacent
    if (d->u_st != 1 || d->u_sd < d->T) return NAJU_E_STRIDE;
  } else if (d->u_sd < 0 || d->u_st < d->D) {
    return NAJU_E_STRIDE;
  }
  if (d->fl_st < d->D || d->il_st < d->D) return NAJU_E_STRIDE;
  if (d->bm_st < d->N || d->cm_st < d->N) return NAJU_E_STRIDE;
  if (d->u_sb < 0 || d->fl_sb < 0 || d->il_sb < 0 || d->bm_sb < 0 || d->cm_sb < 0) return NAJU_E_STRIDE;
  return NAJU_OK;
}

template <typename P>
void fill_common(P& p, const naju_scan_desc* d, const Geometry& g) {
  p.B = d->B; p.T = d->T; p.D = d->D; p.N = d->N;
  p.nchunks = g.nchunks; p.ndt = g.ndt; p.bc_dtype = d->bc_dtype;
  p.u_sb = d->u_sb; p.u_st = d->u_st; p.fl_sb = d->fl_sb; p.fl_st = d->fl_st;
  p.il_sb = d->il_sb; p.il_st = d->il_st; p.bm_sb = d->bm_sb; p.bm_st = d->bm_st;
  p.cm_sb = d->cm_sb; p.cm_st = d->cm_st;
  p.u_sd = d->u_sd > 1 ? d->u_sd : 1;
}

__global__ void copy_state_kernel(const float* __restrict__ src, float* __restrict__ dst, int64_t n,
                                  float fill) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = src ? src[i] : fill;
}

// Makes a device-side failure loud without a host round trip.  Runs after the kernels of a call,
// on the same stream: when the call's status word is non-zero (a bounded wait ran out), or the
// forward that wrote these checkpoints failed that way, every output of the call is overwritten
// with all-ones bytes (NaN in fp32, bf16 and fp16 alike).  In the normal case it reads two words
// and returns.
struct PoisonList {
  void* ptr[8];
  unsigned long long bytes[8];
  int n;
};

__global__ void poison_on_failure_kernel(ScratchHeader* hdr, int* fwd_form, int mark_trailer, int inject,
                                         PoisonList list) {
  __shared__ int s_bad;
  if (threadIdx.x == 0) {
    if (inject && blockIdx.x == 0) atomicOr(&hdr->status, NAJU_ST_LOOKBACK_TIMEOUT);
    int st = *reinterpret_cast<volatile int*>(&hdr->status);
    if (inject) st |= NAJU_ST_LOOKBACK_TIMEOUT;
    const int failed_before = (!mark_trailer && fwd_form != nullptr) ? (*fwd_form & 4) : 0;
    s_bad = (st != 0 || failed_before != 0) ? 1 : 0;
    if (s_bad && mark_trailer && fwd_form != nullptr && blockIdx.x == 0) atomicOr(fwd_form, 4);
  }
  __syncthreads();
  if (!s_bad) return;
  for (int k = 0; k < list.n; ++k) {
    unsigned char* p = static_cast<unsigned char*>(list.ptr[k]);
    const unsigned long long nb = list.bytes[k];
    for (unsigned long long i = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nb;
         i += static_cast<unsigned long long>(gridDim.x) * blockDim.x)
      p[i] = 0xFF;
  }
}

void poison_add(PoisonList& l, void* p, size_t bytes) {
  if (p != nullptr && bytes > 0 && l.n < 8) {
    l.ptr[l.n] = p;
    l.bytes[l.n] = bytes;
    ++l.n;
  }
}

int launch_poison(ScratchHeader* hdr, int* fwd_form, bool mark_trailer, bool inject, const PoisonList& l,
                  cudaStream_t st) {
  poison_on_failure_kernel<<<64, 256, 0, st>>>(hdr, fwd_form, mark_trailer ? 1 : 0, inject ? 1 : 0, l);
  return static_cast<int>(cudaGetLastError());
}

int read_header_word(const void* scratch, size_t offset, void* stream) {
  if (!scratch) return NAJU_E_NULL;
  int word = 0;
  cudaError_t e = cudaMemcpyAsync(&word, static_cast<const char*>(scratch) + offset, sizeof(int),
                                  cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return static_cast<int>(e);
  return word;
}

}  // namespace

extern "C" {

int naju_b200_version(void) { return NAJU_B200_ABI_VERSION; }

const char* naju_b200_strerror(int code) {
  switch (code) {
    case NAJU_OK: return "ok";
    case NAJU_E_NULL: return "a required pointer is NULL";
    case NAJU_E_SHAPE: return "shape out of range (need B,T,D >= 0 and 1 <= N <= 128)";
    case NAJU_E_DTYPE: return "unsupported dtype combination (gates must match u or be fp32)";
    case NAJU_E_STRIDE: return "unsupported strides (inner stride 1, row stride >= row length)";
    case NAJU_E_WORKSPACE: return "workspace missing or not 256-byte aligned";
    case NAJU_E_ALIGN: return "pointer not aligned to its element size";
    case NAJU_E_UNSUPPORTED:
      return "NAJU_FLAG_CHUNKED_ONLY: no tensor-core kernel takes this problem (needs 16-bit u, bf16 B/C, "
             "N == 16, T > 0 and strides that are multiples of 16 bytes)";
    case NAJU_E_TOO_LARGE:
      return "problem too large for the built-in workspace of naju_b200_fwd_noalloc (32 MiB); "
             "use naju_b200_fwd with caller-owned workspaces";
    default: return code > 0 ? cudaGetErrorString(static_cast<cudaError_t>(code)) : "unknown error";
  }
}

int naju_b200_chunk_len(const naju_scan_desc* desc) {
  if (check_desc(desc, false) != NAJU_OK) return 0;
  return chunk_len_for(padded_states(desc->N));
}

size_t naju_b200_ckpt_bytes(const naju_scan_desc* desc) {
  if (check_desc(desc, true) != NAJU_OK) return 0;
  return ckpt_layout(make_geometry(*desc)).bytes;
}

size_t naju_b200_ckpt_decay_offset(const naju_scan_desc* desc) {
  if (check_desc(desc, true) != NAJU_OK) return 0;
  return ckpt_layout(make_geometry(*desc)).off_P;
}

size_t naju_b200_fwd_scratch_bytes(const naju_scan_desc* desc) {
  if (check_desc(desc, true) != NAJU_OK) return 0;
  return fwd_scratch_layout(make_geometry(*desc)).bytes;
}

size_t naju_b200_bwd_scratch_bytes(const naju_scan_desc* desc) {
  if (check_desc(desc, true) != NAJU_OK) return 0;
  return bwd_scratch_layout(make_geometry(*desc)).bytes;
}

int naju_b200_fwd(const naju_scan_desc* desc, const void* u, const void* f_logit,
                  const void* i_logit, const void* Bm, const void* Cm, const float* D_skip,
                  const float* h0, void* y, float* hT, float* pT, void* ckpt, void* scratch,
                  void* stream) {
  int rc = check_desc(desc, true);
  if (rc != NAJU_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t nstate = static_cast<int64_t>(desc->B) * desc->D * desc->N;
  const int64_t nchan = static_cast<int64_t>(desc->B) * desc->D;
  if (desc->B == 0 || desc->D == 0) return NAJU_OK;
  if (desc->T == 0) {  // empty time axis: the state passes through unchanged
    if (hT) copy_state_kernel<<<static_cast<unsigned>((nstate + 255) / 256), 256, 0, st>>>(h0, hT, nstate, 0.f);
    if (pT) copy_state_kernel<<<static_cast<unsigned>((nchan + 255) / 256), 256, 0, st>>>(nullptr, pT, nchan, 1.f);
    return static_cast<int>(cudaGetLastError());
  }
  if (!u || !f_logit || !i_logit || !Bm || !Cm || !D_skip || !y) return NAJU_E_NULL;
  if (!ckpt || !scratch || !aligned(ckpt, 256) || !aligned(scratch, 256)) return NAJU_E_WORKSPACE;
  if ((rc = check_strides(desc)) != NAJU_OK) return rc;
  if (!aligned(u, dtype_size(desc->act_dtype)) || !aligned(y, dtype_size(desc->act_dtype)) ||
      !aligned(f_logit, dtype_size(desc->gate_dtype)) || !aligned(i_logit, dtype_size(desc->gate_dtype)) ||
      !aligned(Bm, dtype_size(desc->bc_dtype)) || !aligned(Cm, dtype_size(desc->bc_dtype)))
    return NAJU_E_ALIGN;

  const Geometry g = make_geometry(*desc);
  const CkptLayout cl = ckpt_layout(g);
  const FwdScratchLayout sl = fwd_scratch_layout(g);
  char* ck = static_cast<char*>(ckpt);
  char* sc = static_cast<char*>(scratch);
  cudaError_t e = cudaMemsetAsync(sc, 0, sl.zero_bytes, st);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaMemsetAsync(ck + cl.off_trailer, 0, 256, st);
  if (e != cudaSuccess) return static_cast<int>(e);

  FwdParams p;
  fill_common(p, desc, g);
  p.u = u; p.fl = f_logit; p.il = i_logit; p.Bm = Bm; p.Cm = Cm; p.Dskip = D_skip; p.h0 = h0;
  p.y = y; p.hT = hT; p.pT = pT;
  p.ckS = reinterpret_cast<float*>(ck + cl.off_S);
  p.ckP = reinterpret_cast<float*>(ck + cl.off_P);
  p.fwd_form = reinterpret_cast<int*>(ck + cl.off_trailer);
  p.hdr = reinterpret_cast<ScratchHeader*>(sc);
  p.flags = reinterpret_cast<int*>(sc + sl.off_flags);
  p.aggP = reinterpret_cast<float*>(sc + sl.off_aggP);
  p.aggS = reinterpret_cast<float*>(sc + sl.off_aggS);
  int rck = -1000;
  if (!(desc->flags & NAJU_FLAG_RECURRENT_ONLY)) {
    rck = launch_fwd_tc3(p, g, desc->act_dtype, desc->gate_dtype, desc->bc_dtype, stream);
    // (the ticket kernel reads u channel-contiguous only; a time-contiguous u that the walk kernel
    // declines goes to the recurrent kernel, which transposes its tile while staging it)
    if (rck == -1000 && p.u_sd == 1)
      rck = launch_fwd_tc2(p, g, desc->act_dtype, desc->gate_dtype, desc->bc_dtype, stream);
    if (rck == -1000 && (desc->flags & NAJU_FLAG_CHUNKED_ONLY)) return NAJU_E_UNSUPPORTED;
  }
  if (rck == -1000) rck = launch_fwd_simt(p, g, desc->act_dtype, desc->gate_dtype, stream);
  if (rck != 0) return rck;
  PoisonList pl = {};
  poison_add(pl, y, static_cast<size_t>(desc->B) * desc->T * desc->D * dtype_size(desc->act_dtype));
  poison_add(pl, hT, static_cast<size_t>(nstate) * 4);
  poison_add(pl, pT, static_cast<size_t>(nchan) * 4);
  return launch_poison(p.hdr, p.fwd_form, true, (desc->flags & NAJU_FLAG_INJECT_TIMEOUT) != 0, pl, st);
}

int naju_b200_bwd(const naju_scan_desc* desc, const void* u, const void* f_logit,
                  const void* i_logit, const void* Bm, const void* Cm, const float* D_skip,
                  const float* h0, const void* dy, const float* dhT, const void* ckpt, void* du,
                  void* dfl, void* dil, void* dB, void* dC, float* dD, float* dh0, void* scratch,
                  void* stream) {
  int rc = check_desc(desc, true);
  if (rc != NAJU_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (desc->B == 0 || desc->D == 0) return NAJU_OK;
  if (desc->T == 0) {  // nothing to differentiate: dh0 = dhT, dD = 0
    const int64_t nstate = static_cast<int64_t>(desc->B) * desc->D * desc->N;
    if (dh0) copy_state_kernel<<<static_cast<unsigned>((nstate + 255) / 256), 256, 0, st>>>(dhT, dh0, nstate, 0.f);
    if (dD) copy_state_kernel<<<static_cast<unsigned>((desc->D + 255) / 256), 256, 0, st>>>(nullptr, dD, desc->D, 0.f);
    return static_cast<int>(cudaGetLastError());
  }
  if (!u || !f_logit || !i_logit || !Bm || !Cm || !D_skip || !dy || !du || !dfl || !dil || !dB ||
      !dC || !dD)
    return NAJU_E_NULL;
  if (!ckpt || !scratch || !aligned(ckpt, 256) || !aligned(scratch, 256)) return NAJU_E_WORKSPACE;
  if ((rc = check_strides(desc)) != NAJU_OK) return rc;

  const Geometry g = make_geometry(*desc);
  const CkptLayout cl = ckpt_layout(g);
  const BwdScratchLayout sl = bwd_scratch_layout(g);
  const char* ck = static_cast<const char*>(ckpt);
  char* sc = static_cast<char*>(scratch);
  cudaError_t e = cudaMemsetAsync(sc, 0, sl.zero_bytes, st);
  if (e != cudaSuccess) return static_cast<int>(e);

  BwdParams p;
  fill_common(p, desc, g);
  p.u = u; p.fl = f_logit; p.il = i_logit; p.Bm = Bm; p.Cm = Cm; p.dy = dy; p.Dskip = D_skip;
  p.h0 = h0; p.dhT = dhT;
  p.ckS = reinterpret_cast<const float*>(ck + cl.off_S);
  p.du = du; p.dfl = dfl; p.dil = dil; p.dh0 = dh0;
  p.hdr = reinterpret_cast<ScratchHeader*>(sc);
  p.flags = reinterpret_cast<int*>(sc + sl.off_flags);
  p.aggP = reinterpret_cast<float*>(sc + sl.off_aggP);
  p.aggL = reinterpret_cast<float*>(sc + sl.off_aggL);
  p.inclL = reinterpret_cast<float*>(sc + sl.off_inclL);
  p.dBpart = reinterpret_cast<float*>(sc + sl.off_dBpart);
  p.dCpart = reinterpret_cast<float*>(sc + sl.off_dCpart);
  p.dDpart = reinterpret_cast<float*>(sc + sl.off_dDpart);
  p.fwd_form = reinterpret_cast<const int*>(ck + cl.off_trailer);
  p.tc_launched = 0;
  if (!(desc->flags & NAJU_FLAG_RECURRENT_ONLY)) {
    // The tensor-core backward stands down on the device unless the forward of these inputs ran
    // chunked and met no deep-gate tile; the recurrent backward launched after it does the
    // opposite, so exactly one of the two does the work and no host round trip is needed.
    const int rc2 = launch_bwd_tc(p, g, desc->act_dtype, desc->gate_dtype, desc->bc_dtype, p.fwd_form, stream);
    if (rc2 == 0) p.tc_launched = 1;
    else if (rc2 != -1000) return rc2;
  }
  const int rcs = launch_bwd_simt(p, g, desc->act_dtype, desc->gate_dtype, dB, dC, dD, stream);
  if (rcs != 0) return rcs;
  PoisonList pl = {};
  const size_t ntd = static_cast<size_t>(desc->B) * desc->T * desc->D;
  const size_t ntn = static_cast<size_t>(desc->B) * desc->T * desc->N;
  poison_add(pl, du, ntd * dtype_size(desc->act_dtype));
  poison_add(pl, dfl, ntd * dtype_size(desc->gate_dtype));
  poison_add(pl, dil, ntd * dtype_size(desc->gate_dtype));
  poison_add(pl, dB, ntn * dtype_size(desc->bc_dtype));
  poison_add(pl, dC, ntn * dtype_size(desc->bc_dtype));
  poison_add(pl, dD, static_cast<size_t>(desc->D) * 4);
  poison_add(pl, dh0, static_cast<size_t>(desc->B) * desc->D * desc->N * 4);
  return launch_poison(p.hdr, const_cast<int*>(p.fwd_form), false, (desc->flags & NAJU_FLAG_INJECT_TIMEOUT) != 0, pl, st);
}

int naju_b200_step(const naju_scan_desc* desc, float* state, const void* u, const void* f_logit,
                   const void* i_logit, const void* Bm, const void* Cm, const float* D_skip,
                   void* y, void* stream) {
  int rc = check_desc(desc, false);
  if (rc != NAJU_OK) return rc;
  if (desc->B == 0 || desc->D == 0) return NAJU_OK;
  if (!state || !u || !f_logit || !i_logit || !Bm || !Cm || !D_skip || !y) return NAJU_E_NULL;
  if (desc->u_sb < desc->D || desc->fl_sb < desc->D || desc->il_sb < desc->D ||
      desc->bm_sb < desc->N || desc->cm_sb < desc->N)
    return NAJU_E_STRIDE;
  if (!aligned(state, 16)) return NAJU_E_ALIGN;
  return launch_step(*desc, state, u, f_logit, i_logit, Bm, Cm, D_skip, y, stream);
}

int naju_b200_read_status(const void* scratch, void* stream) {
  return read_header_word(scratch, offsetof(ScratchHeader, status), stream);
}

int naju_b200_read_form(const void* scratch, void* stream) {
  return read_header_word(scratch, offsetof(ScratchHeader, form), stream);
}

}  // extern "C"
