/* naju_b200 — C ABI of the B200 (sm_100a) gated diagonal state-space scan.
 *
 * This is the drop-in boundary for the scan path of the Naju reference project:
 * every entry point below replaces one of the calls its scan backends make into
 * native code.  Reference citations are paths inside that project.
 *
 * Conventions
 *  - All pointers are DEVICE pointers unless the name ends in _host.
 *  - The library never allocates or frees device memory: the caller sizes
 *    workspaces with the *_bytes() queries and owns every buffer.
 *  - Every call is asynchronous on `stream` (a cudaStream_t passed as void*).
 *  - Return value: 0 = ok, negative = rejected argument (NAJU_E_*), positive =
 *    CUDA runtime error code of the failed launch.  Device-side conditions (a
 *    bounded wait that ran out) are recorded in the workspace status word and
 *    read back with naju_b200_read_status().  They are never silent: a call whose
 *    status word ends non-zero overwrites its own outputs with NaN before it
 *    completes (on the device, no host synchronisation), and a backward given the
 *    checkpoints of such a forward does the same.
 *  - Shapes follow naju/scan.py:3-12: u, f_logit, i_logit, y [B,T,D];
 *    Bm, Cm [B,T,N]; D_skip [D]; states [B,D,N] fp32.  The sigmoid of both gate
 *    logits is applied inside (naju/scan.py:81-82).
 */
#ifndef NAJU_B200_H_
#define NAJU_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NAJU_B200_ABI_VERSION 2

/* element types of caller tensors */
enum { NAJU_F32 = 0, NAJU_BF16 = 1, NAJU_F16 = 2 };

/* argument errors */
enum {
  NAJU_OK = 0,
  NAJU_E_NULL = -1,      /* a required pointer is NULL */
  NAJU_E_SHAPE = -2,     /* B,T,D,N out of range (N must be 1..128, as naju/cuda/naju_cuda.cu:222) */
  NAJU_E_DTYPE = -3,     /* unsupported dtype combination */
  NAJU_E_STRIDE = -4,    /* inner stride not 1 / row stride smaller than the row */
  NAJU_E_WORKSPACE = -5, /* workspace too small or misaligned */
  NAJU_E_ALIGN = -6,     /* a pointer is not aligned to its element size */
  NAJU_E_TOO_LARGE = -7, /* problem needs more workspace than naju_b200_fwd_noalloc() owns */
  NAJU_E_UNSUPPORTED = -8 /* NAJU_FLAG_CHUNKED_ONLY was set and no tensor-core kernel takes the problem */
};

/* device-side status bits, OR-ed into the workspace status word */
enum {
  NAJU_ST_LOOKBACK_TIMEOUT = 1, /* a bounded wait on a neighbouring chunk's carry ran out */
  NAJU_ST_BAD_TILE = 2,         /* internal tile index out of range (never expected) */
  NAJU_ST_MMA_TIMEOUT = 4,      /* a bounded wait on a tensor-core completion barrier ran out */
  NAJU_ST_DEEP_TILE = 8         /* the tensor-core backward met a deep-gate tile (never expected:
                                   the forward routes such problems to the recurrent backward) */
};

/* desc->flags */
enum {
  NAJU_FLAG_RECURRENT_ONLY = 1, /* always take the exact recurrent kernels, never the
                                   tensor-core chunked form */
  NAJU_FLAG_CHUNKED_ONLY = 2,   /* forward: fail with NAJU_E_UNSUPPORTED instead of falling back
                                   when no tensor-core kernel takes the problem (ignored by the
                                   backward, whose kernel follows from how the forward ran) */
  NAJU_FLAG_INJECT_TIMEOUT = 4  /* fault injection for tests: behave as if a bounded device-side
                                   wait had run out (sets NAJU_ST_LOOKBACK_TIMEOUT after the
                                   kernels; nothing on the device actually waits or hangs) */
};

/* which kernel family did the work of a call (naju_b200_read_form) */
enum {
  NAJU_FORM_NONE = 0,      /* nothing ran (empty problem) */
  NAJU_FORM_RECURRENT = 1, /* exact recurrent kernels */
  NAJU_FORM_TC_TICKET = 2, /* tensor-core chunked forward, tiles by ticket with look-back carry */
  NAJU_FORM_TC_WALK = 3    /* tensor-core chunked form walking each channel tile along time
                              (forward) or in reverse time (backward) */
};

/* Problem description shared by forward and backward.
 * Strides are in ELEMENTS.  The innermost (channel / state) stride of every
 * tensor is 1.  u/f_logit/i_logit may each have their own batch and time
 * strides (the mixer hands Bm and Cm as two views of one [B,T,2N] tensor,
 * naju/mixer.py:116, so their time stride is 2N there).
 * One exception: u may be TIME-contiguous -- the [B,D,T] memory the mixer's depthwise
 * convolution leaves behind, viewed as [B,T,D] (naju/mixer.py:115).  Then u_st = 1 and
 * u_sd > 1 is the element stride between channels; element (b,t,d) of u sits at
 * b*u_sb + t + d*u_sd.  u_sd = 0 or 1 means the usual channel-contiguous u.  The backward then
 * writes du with u's strides (the gradient of a [B,D,T] tensor is wanted in [B,D,T] memory);
 * every other tensor keeps its channel-contiguous layout. */
typedef struct naju_scan_desc {
  int32_t B, T, D, N;
  int32_t act_dtype;  /* u, y, dy, du            */
  int32_t gate_dtype; /* f_logit, i_logit, and their gradients */
  int32_t bc_dtype;   /* Bm, Cm, dB, dC          */
  int32_t flags;      /* NAJU_FLAG_* bits        */
  int64_t u_sb, u_st;
  int64_t fl_sb, fl_st;
  int64_t il_sb, il_st;
  int64_t bm_sb, bm_st;
  int64_t cm_sb, cm_st;
  int64_t u_sd;       /* 0 / 1: u is channel-contiguous; > 1: time-contiguous u, see above */
} naju_scan_desc;

/* ABI version of the loaded library (NAJU_B200_ABI_VERSION it was built with). */
int naju_b200_version(void);

/* Human-readable text for a return code of this library. */
const char* naju_b200_strerror(int code);

/* Time steps per chunk of the forward/backward kernels for this problem (the spacing of
 * the saved chunk-boundary states). */
int naju_b200_chunk_len(const naju_scan_desc* desc);

/* Bytes of the chunk-boundary state buffer the forward writes and the backward reads
 * (the counterpart of the `ckpt` tensor of naju/cuda/naju_cuda.cu:45-46,246). */
size_t naju_b200_ckpt_bytes(const naju_scan_desc* desc);

/* Byte offset, inside the checkpoint buffer, of the cumulative retention products
 * P[chunk][b][channel tile][128] fp32 (product of the retention gate from t=0 to the end of
 * each chunk; padded channels included).  The chunk-end states [chunk][b][tile][128][NS] fp32
 * start at offset 0, NS = N rounded up to 16, 32, 64 or 128. */
size_t naju_b200_ckpt_decay_offset(const naju_scan_desc* desc);

/* Bytes of transient scratch for one forward / one backward call. */
size_t naju_b200_fwd_scratch_bytes(const naju_scan_desc* desc);
size_t naju_b200_bwd_scratch_bytes(const naju_scan_desc* desc);

/* Forward scan.  Replaces ext.fwd / ext.fwd_chunked (naju/cuda/naju_cuda.cu:217-259,
 * naju/cuda/__init__.py:48-54) and the Triton forwards (naju/chunk_triton.py:147-181,
 * naju/chunk_affine_triton.py:256-290).
 *   h0     optional [B,D,N] fp32 initial state (NULL = zeros, the reference behaviour)
 *   y      [B,T,D] contiguous, act_dtype
 *   hT     optional [B,D,N] fp32 final state
 *   pT     optional [B,D] fp32 product of the retention gate over all T steps
 *   ckpt   naju_b200_ckpt_bytes() bytes, 256-byte aligned; keep it for the backward
 *   scratch naju_b200_fwd_scratch_bytes() bytes, 256-byte aligned; dead when the call has run
 */
int naju_b200_fwd(const naju_scan_desc* desc, const void* u, const void* f_logit,
                  const void* i_logit, const void* Bm, const void* Cm, const float* D_skip,
                  const float* h0, void* y, float* hT, float* pT, void* ckpt, void* scratch,
                  void* stream);

/* Backward scan: all gradients in one pass over the sequence in reverse time.
 * Replaces ext.bwd (naju/cuda/naju_cuda.cu:261-286) and naju_chunk_backward
 * (naju/chunk_bwd_triton.py:187-243).
 *   ckpt   the buffer the forward of the SAME inputs filled
 *   dy     [B,T,D] contiguous act_dtype;  dhT optional [B,D,N] fp32 adjoint of hT
 *   du [B,T,D] act_dtype; dfl, dil [B,T,D] gate_dtype; dB, dC [B,T,N] bc_dtype; all contiguous
 *   dD [D] fp32;  dh0 optional [B,D,N] fp32
 */
int naju_b200_bwd(const naju_scan_desc* desc, const void* u, const void* f_logit,
                  const void* i_logit, const void* Bm, const void* Cm, const float* D_skip,
                  const float* h0, const void* dy, const float* dhT, const void* ckpt,
                  void* du, void* dfl, void* dil, void* dB, void* dC, float* dD, float* dh0,
                  void* scratch, void* stream);

/* Single-token recurrent update for decode (one iteration of naju/scan.py:87-91; the
 * reference has no such entry point).  state [B,D,N] fp32 is updated in place.
 *   u, f_logit, i_logit, y : [B,D] with batch strides u_sb/fl_sb/il_sb (time strides unused)
 *   Bm, Cm : [B,N] with batch strides bm_sb/cm_sb;  desc->T is ignored.
 */
int naju_b200_step(const naju_scan_desc* desc, float* state, const void* u, const void* f_logit,
                   const void* i_logit, const void* Bm, const void* Cm, const float* D_skip,
                   void* y, void* stream);

/* Size of the built-in workspace of naju_b200_fwd_noalloc(): 32 MiB of device memory that
 * every GPU loading this library holds until the process exits. */
#define NAJU_B200_NOALLOC_BYTES (32u << 20)

/* Forward scan for callers that cannot allocate device memory.  (No counterpart in the
 * reference, whose native ops allocate their own outputs and checkpoints.)
 *
 * Meant for hosts that give a plugin only its input and output buffers and forbid allocation
 * on that path -- an inference engine's enqueue hook, a serving loop that reserved its memory
 * at start-up -- because cudaMalloc synchronises the device and can fail when memory is short.
 * Same arguments and results as naju_b200_fwd() minus the two workspaces (and minus pT): they
 * are carved out of a NAJU_B200_NOALLOC_BYTES array inside the library.  Nothing is allocated
 * or freed by this call.
 *   - Problems with naju_b200_ckpt_bytes() + naju_b200_fwd_scratch_bytes() above that size
 *     are rejected with NAJU_E_TOO_LARGE (B*T*D up to about 15 M token-channels at
 *     N <= 16 fits).
 *   - The first call on each device looks the array's address up (with that device current).
 *     With lazy module loading that is also when the array gets its device memory, so this one
 *     call may take milliseconds and can fail on a device that is already full: make it once
 *     per device at start-up, outside any stream capture.  The address is cached per device and
 *     does not survive cudaDeviceReset().
 *   - Device-side status and kernel form of the last call: naju_b200_noalloc_read_status(),
 *     naju_b200_noalloc_read_form() (the scratch header is at the start of the array).
 *   - All calls on a device share the array: calls that may overlap on the GPU (different
 *     streams, or this and another thread) race on it and must be serialised by the caller.
 *     The array keeps the previous call's contents; the call clears the part that has to
 *     start at zero itself.
 *   - The chunk-boundary states stay inside the library, so there is no matching backward:
 *     use it for inference (prefill) only.
 */
int naju_b200_fwd_noalloc(const naju_scan_desc* desc, const void* u, const void* f_logit,
                          const void* i_logit, const void* Bm, const void* Cm,
                          const float* D_skip, const float* h0, void* y, float* hT, void* stream);

/* Synchronises `stream` and returns the status word of a scratch buffer a forward or
 * backward call used (0 = clean; NAJU_ST_* bits otherwise), or a negative/positive error
 * code as above. */
int naju_b200_read_status(const void* scratch, void* stream);

/* Synchronises `stream` and returns which kernel family did the work of the forward or
 * backward call that used this scratch buffer (NAJU_FORM_*), or a negative/positive error code.
 * The reference picks its kernels on the host (naju/scan.py:48-72); here part of the choice is
 * made on the device, and this is how a caller or a test sees it. */
int naju_b200_read_form(const void* scratch, void* stream);

/* The same two queries for the built-in workspace of naju_b200_fwd_noalloc() on the current
 * device (the caller has no pointer to it).  No counterpart in the reference. */
int naju_b200_noalloc_read_status(void* stream);
int naju_b200_noalloc_read_form(void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NAJU_B200_H_ */
