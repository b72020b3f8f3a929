// Host/device parameter blocks and workspace layouts of the scan kernels.
#pragma once

#include <stddef.h>
#include <stdint.h>

#include "naju_b200.h"

namespace naju {

// Padded state width: the kernels are instantiated for these widths and pad B/C with zeros.
inline int padded_states(int N) { return N <= 16 ? 16 : N <= 32 ? 32 : N <= 64 ? 64 : 128; }
// Chunk length (time steps per tile); the spacing of the saved chunk-boundary states.
inline int chunk_len_for(int NS) { return NS <= 32 ? 64 : 32; }

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

struct Geometry {
  int B, T, D, N, NS, TC, nchunks, ndt;
  int64_t ntiles;  // nchunks * B * ndt
};

inline Geometry make_geometry(const naju_scan_desc& d) {
  Geometry g;
  g.B = d.B; g.T = d.T; g.D = d.D; g.N = d.N;
  g.NS = padded_states(d.N);
  g.TC = chunk_len_for(g.NS);
  g.nchunks = (d.T + g.TC - 1) / g.TC;
  g.ndt = (d.D + 127) / 128;
  g.ntiles = static_cast<int64_t>(g.nchunks) * d.B * g.ndt;
  return g;
}

// Checkpoint buffer (persists from forward to backward):
//   stateS [ntiles][128][NS] fp32  state at the END of each chunk (tile = (chunk, b, dtile))
//   stateP [ntiles][128]     fp32  product of the retention gate from t=0 to the chunk end
// Trailer of the checkpoint buffer: how the forward ran, for the backward's kernel choice.
//   bit 0  the forward ran in the tensor-core chunked form, walking each channel tile in time
//   bit 1  it met at least one deep-gate tile (the factorised backward cannot take those)
//   bit 2  a bounded wait of the forward ran out: its outputs were overwritten with NaN, and the
//          backward of these checkpoints does the same to its own
struct CkptTrailer {
  int fwd_form;
};

struct CkptLayout {
  size_t off_S, off_P, off_trailer, bytes;
};
inline CkptLayout ckpt_layout(const Geometry& g) {
  CkptLayout l;
  l.off_S = 0;
  l.off_P = align_up(static_cast<size_t>(g.ntiles) * 128 * g.NS * 4, 256);
  l.off_trailer = l.off_P + align_up(static_cast<size_t>(g.ntiles) * 128 * 4, 256);
  l.bytes = l.off_trailer + 256;
  return l;
}

// Scratch header, first 256 bytes of every scratch buffer.
struct ScratchHeader {
  int status;            // NAJU_ST_* bits
  unsigned int ticket;   // dynamic tile counter
  int form;              // NAJU_FORM_* of the kernel that did the work (written by that kernel)
};

// Forward scratch: header | flags[ntiles] | aggP[ntiles][128] | aggS[ntiles][128][NS]
struct FwdScratchLayout {
  size_t off_flags, off_aggP, off_aggS, bytes, zero_bytes;
};
inline FwdScratchLayout fwd_scratch_layout(const Geometry& g) {
  FwdScratchLayout l;
  l.off_flags = 256;
  l.zero_bytes = l.off_flags + align_up(static_cast<size_t>(g.ntiles) * 4, 256);
  l.off_aggP = l.zero_bytes;
  l.off_aggS = l.off_aggP + align_up(static_cast<size_t>(g.ntiles) * 128 * 4, 256);
  l.bytes = l.off_aggS + align_up(static_cast<size_t>(g.ntiles) * 128 * g.NS * 4, 256);
  return l;
}

// Backward scratch: header | flags | aggP | aggL | inclL | dBpart,dCpart [B][T][ndt][NS] |
// dDpart [nchunks*B][ndt*128]
struct BwdScratchLayout {
  size_t off_flags, off_aggP, off_aggL, off_inclL, off_dBpart, off_dCpart, off_dDpart, bytes,
      zero_bytes;
};
inline BwdScratchLayout bwd_scratch_layout(const Geometry& g) {
  BwdScratchLayout l;
  l.off_flags = 256;
  l.zero_bytes = l.off_flags + align_up(static_cast<size_t>(g.ntiles) * 4, 256);
  l.off_aggP = l.zero_bytes;
  const size_t sP = align_up(static_cast<size_t>(g.ntiles) * 128 * 4, 256);
  const size_t sS = align_up(static_cast<size_t>(g.ntiles) * 128 * g.NS * 4, 256);
  const size_t sBC = align_up(static_cast<size_t>(g.B) * g.T * g.ndt * g.NS * 4, 256);
  const size_t sD = align_up(static_cast<size_t>(g.nchunks) * g.B * g.ndt * 128 * 4, 256);
  l.off_aggL = l.off_aggP + sP;
  l.off_inclL = l.off_aggL + sS;
  l.off_dBpart = l.off_inclL + sS;
  l.off_dCpart = l.off_dBpart + sBC;
  l.off_dDpart = l.off_dCpart + sBC;
  l.bytes = l.off_dDpart + sD;
  return l;
}

struct FwdParams {
  const void *u, *fl, *il, *Bm, *Cm;
  const float* Dskip;
  const float* h0;
  void* y;
  float* hT;
  float* pT;
  float* ckS;
  float* ckP;
  int* fwd_form;  // CkptTrailer::fwd_form
  ScratchHeader* hdr;
  int* flags;
  float* aggP;
  float* aggS;
  int B, T, D, N, nchunks, ndt, bc_dtype;
  int64_t u_sb, u_st, fl_sb, fl_st, il_sb, il_st, bm_sb, bm_st, cm_sb, cm_st;
  int64_t u_sd;  // element stride between channels of u: 1, or > 1 for a time-contiguous u (then u_st == 1)
};

struct BwdParams {
  const void *u, *fl, *il, *Bm, *Cm, *dy;
  const float* Dskip;
  const float* h0;
  const float* dhT;
  const float* ckS;
  const int* fwd_form;  // CkptTrailer::fwd_form; when (fwd_form & 3) == 1 the tensor-core backward runs
  int tc_launched;      // the tensor-core backward was launched for this call (host decision)
  void *du, *dfl, *dil;
  float* dh0;
  ScratchHeader* hdr;
  int* flags;
  float* aggP;
  float* aggL;
  float* inclL;
  float* dBpart;
  float* dCpart;
  float* dDpart;
  int B, T, D, N, nchunks, ndt, bc_dtype;
  int64_t u_sb, u_st, fl_sb, fl_st, il_sb, il_st, bm_sb, bm_st, cm_sb, cm_st;
  int64_t u_sd;  // element stride between channels of u: 1, or > 1 for a time-contiguous u (then u_st == 1)
};

// launchers implemented in the .cu files; return a CUDA runtime error code (0 = ok)
int launch_fwd_simt(const FwdParams& p, const Geometry& g, int act_dtype, int gate_dtype,
                    void* stream);
// TMA-fed persistent tensor-core forward; returns -1000 when the problem cannot take it
int launch_fwd_tc2(const FwdParams& p, const Geometry& g, int act_dtype, int gate_dtype, int bc_dtype,
                   void* stream);
// walk-along-time tensor-core forward (two threads per channel); -1000 when it cannot take the problem
int launch_fwd_tc3(const FwdParams& p, const Geometry& g, int act_dtype, int gate_dtype, int bc_dtype,
                   void* stream);
int launch_bwd_simt(const BwdParams& p, const Geometry& g, int act_dtype, int gate_dtype,
                    void* dB, void* dC, float* dD, void* stream);
// tensor-core backward; returns -1000 when the problem cannot take it
int launch_bwd_tc(const BwdParams& p, const Geometry& g, int act_dtype, int gate_dtype, int bc_dtype,
                  const int* fwd_form, void* stream);
int launch_step(const naju_scan_desc& d, float* state, const void* u, const void* fl,
                const void* il, const void* Bm, const void* Cm, const float* Dskip, void* y,
                void* stream);

}  // namespace naju
