"""ctypes binding of libnaju_b200.so (the C ABI declared in include/naju_b200.h).

There is no fallback: if the library has not been built, or the caller's tensors are not on
a CUDA device, the functions here raise.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnaju_b200.so")

NAJU_F32, NAJU_BF16, NAJU_F16 = 0, 1, 2
ABI_VERSION = 2

ST_LOOKBACK_TIMEOUT = 1
ST_BAD_TILE = 2
ST_MMA_TIMEOUT = 4
ST_DEEP_TILE = 8
FLAG_RECURRENT_ONLY = 1
FLAG_CHUNKED_ONLY = 2
FLAG_INJECT_TIMEOUT = 4
FORM_NONE, FORM_RECURRENT, FORM_TC_TICKET, FORM_TC_WALK = 0, 1, 2, 3
E_TOO_LARGE = -7
E_UNSUPPORTED = -8
NOALLOC_BYTES = 32 << 20

# every symbol include/naju_b200.h declares
EXPORTS = ("naju_b200_version", "naju_b200_strerror", "naju_b200_chunk_len",
           "naju_b200_ckpt_bytes", "naju_b200_ckpt_decay_offset", "naju_b200_fwd_scratch_bytes", "naju_b200_bwd_scratch_bytes",
           "naju_b200_fwd", "naju_b200_bwd", "naju_b200_step", "naju_b200_read_status",
           "naju_b200_fwd_noalloc", "naju_b200_read_form", "naju_b200_noalloc_read_status",
           "naju_b200_noalloc_read_form")


class ScanDesc(ctypes.Structure):
    """Mirror of struct naju_scan_desc."""
    _fields_ = [("B", ctypes.c_int32), ("T", ctypes.c_int32), ("D", ctypes.c_int32),
                ("N", ctypes.c_int32), ("act_dtype", ctypes.c_int32),
                ("gate_dtype", ctypes.c_int32), ("bc_dtype", ctypes.c_int32),
                ("flags", ctypes.c_int32),
                ("u_sb", ctypes.c_int64), ("u_st", ctypes.c_int64),
                ("fl_sb", ctypes.c_int64), ("fl_st", ctypes.c_int64),
                ("il_sb", ctypes.c_int64), ("il_st", ctypes.c_int64),
                ("bm_sb", ctypes.c_int64), ("bm_st", ctypes.c_int64),
                ("cm_sb", ctypes.c_int64), ("cm_st", ctypes.c_int64),
                ("u_sd", ctypes.c_int64)]


_lib = None


def load():
    """Loads the shared library once; raises if it is missing or has another ABI version."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m naju_b200.build` "
            "(there is no CPU or PyTorch fallback for the scan)")
    lib = ctypes.CDLL(LIB_PATH)
    vp, dp = ctypes.c_void_p, ctypes.POINTER(ScanDesc)
    lib.naju_b200_version.restype = ctypes.c_int
    lib.naju_b200_version.argtypes = []
    lib.naju_b200_strerror.restype = ctypes.c_char_p
    lib.naju_b200_strerror.argtypes = [ctypes.c_int]
    lib.naju_b200_chunk_len.restype = ctypes.c_int
    lib.naju_b200_chunk_len.argtypes = [dp]
    for name in ("naju_b200_ckpt_bytes", "naju_b200_ckpt_decay_offset", "naju_b200_fwd_scratch_bytes", "naju_b200_bwd_scratch_bytes"):
        getattr(lib, name).restype = ctypes.c_size_t
        getattr(lib, name).argtypes = [dp]
    lib.naju_b200_fwd.restype = ctypes.c_int
    lib.naju_b200_fwd.argtypes = [dp] + [vp] * 13
    lib.naju_b200_bwd.restype = ctypes.c_int
    lib.naju_b200_bwd.argtypes = [dp] + [vp] * 19
    lib.naju_b200_step.restype = ctypes.c_int
    lib.naju_b200_step.argtypes = [dp] + [vp] * 9
    lib.naju_b200_fwd_noalloc.restype = ctypes.c_int
    lib.naju_b200_fwd_noalloc.argtypes = [dp] + [vp] * 10
    for name in ("naju_b200_read_status", "naju_b200_read_form"):
        getattr(lib, name).restype = ctypes.c_int
        getattr(lib, name).argtypes = [vp, vp]
    for name in ("naju_b200_noalloc_read_status", "naju_b200_noalloc_read_form"):
        getattr(lib, name).restype = ctypes.c_int
        getattr(lib, name).argtypes = [vp]
    if lib.naju_b200_version() != ABI_VERSION:
        raise RuntimeError("libnaju_b200.so was built against another ABI version; rebuild it")
    _lib = lib
    return lib


def strerror(code):
    return load().naju_b200_strerror(int(code)).decode()


def check(code, what):
    """Maps a library return code to the exception types the reference raises
    (RuntimeError from TORCH_CHECK, naju/cuda/naju_cuda.cu:220-222)."""
    if code != 0:
        raise RuntimeError(f"{what} failed: {strerror(code)} (code {code})")
