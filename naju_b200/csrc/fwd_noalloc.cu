// Forward scan for callers that must not allocate device memory.
//
// Some hosts hand a plugin nothing but its input and output buffers and forbid it to allocate:
// an inference engine's enqueue hook, or a serving loop that reserved all of its memory at
// start-up.  cudaMalloc is off limits there because it synchronises the whole device and can
// fail once memory is exhausted or fragmented.  naju_b200_fwd() needs two workspaces (the
// chunk-boundary states and the look-back scratch); this entry point takes them from a
// fixed array that is part of the library image instead, so the caller passes only inputs
// and outputs and nothing is allocated, here or in any library this calls.
//
// The price: the array has a fixed size (NAJU_B200_NOALLOC_BYTES; every GPU that loads the
// library holds it until the process exits), larger problems are rejected, and all calls on
// a device share it.
//
// Layout inside the array: the forward's scratch first (so its 256-byte header, with the status
// word, sits at offset 0 whatever the problem size, where naju_b200_noalloc_read_status() finds
// it), then the chunk-boundary states.
//
// The array is part of the library's device image.  With CUDA's lazy module loading that image is
// loaded (and the array backed by device memory) by the first call that touches it on a device,
// so that first call may take milliseconds and may fail when the device is already full: make it
// once per device at start-up, outside any stream capture.  The resolved address is cached per
// device ordinal and does not survive cudaDeviceReset().
#include <cuda_runtime.h>

#include <mutex>

#include "naju_b200.h"

namespace {

// Workspace shared by every naju_b200_fwd_noalloc() call on a device.  In host code this name
// is only a handle of the symbol, not a device address; the address is resolved per device
// with cudaGetSymbolAddress below and that pointer is what the kernels receive.
static __device__ __align__(256) unsigned char g_noalloc_workspace[NAJU_B200_NOALLOC_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
void* g_workspace_addr[kMaxDevices] = {};

size_t align256(size_t x) { return (x + 255) / 256 * 256; }

// Resolves the workspace address on the current device (once per device).
int workspace_for_current_device(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return NAJU_E_SHAPE;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_workspace_addr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_workspace);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (ptr == nullptr) return NAJU_E_WORKSPACE;
    g_workspace_addr[dev] = ptr;
  }
  *out = g_workspace_addr[dev];
  return NAJU_OK;
}

}  // namespace

extern "C" int naju_b200_fwd_noalloc(const naju_scan_desc* desc, const void* u, const void* f_logit,
                                     const void* i_logit, const void* Bm, const void* Cm,
                                     const float* D_skip, const float* h0, void* y, float* hT,
                                     void* stream) {
  if (desc == nullptr) return NAJU_E_NULL;
  if (desc->N < 1 || desc->N > 128 || desc->B < 0 || desc->T < 0 || desc->D < 0) return NAJU_E_SHAPE;
  const size_t ck = naju_b200_ckpt_bytes(desc);
  const size_t sc = align256(naju_b200_fwd_scratch_bytes(desc));
  if (ck + sc > static_cast<size_t>(NAJU_B200_NOALLOC_BYTES)) return NAJU_E_TOO_LARGE;
  void* base = nullptr;
  const int rc = workspace_for_current_device(&base);
  if (rc != NAJU_OK) return rc;
  unsigned char* ws = static_cast<unsigned char*>(base);
  // naju_b200_fwd() clears the part of the scratch that must start at zero (status word, tile
  // ticket, chunk flags) with cudaMemsetAsync on `stream`; everything else is written before it
  // is read, so what the previous call left behind is harmless.
  return naju_b200_fwd(desc, u, f_logit, i_logit, Bm, Cm, D_skip, h0, y, hT, nullptr, ws + sc, ws,
                       stream);
}

// Status word / kernel form of the last naju_b200_fwd_noalloc() call on the current device
// (synchronises `stream`).  A device on which the entry point has not run yet reports 0.
extern "C" int naju_b200_noalloc_read_status(void* stream) {
  void* base = nullptr;
  const int rc = workspace_for_current_device(&base);
  if (rc != NAJU_OK) return rc;
  return naju_b200_read_status(base, stream);
}

extern "C" int naju_b200_noalloc_read_form(void* stream) {
  void* base = nullptr;
  const int rc = workspace_for_current_device(&base);
  if (rc != NAJU_OK) return rc;
  return naju_b200_read_form(base, stream);
}
