"""ctypes front end of the C oracle (TEST INFRASTRUCTURE, never used by the product).

Functions take and return numpy float32 arrays (torch tensors are accepted and
converted); layouts follow naju/scan.py:3-12 of the reference project:
u, f_logit, i_logit [B,T,D]; Bm, Cm [B,T,N]; D_skip [D]; h0 [B,D,N].
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libnaju_oracle.so")
_lib = None


def build(force=False):
    """Compile naju_oracle.c with gcc (OpenMP) next to this file."""
    src = os.path.join(_HERE, "naju_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["gcc", "-O2", "-fopenmp", "-fPIC", "-Wall", "-shared",
                               "-o", _SO, src, "-lm"])
    return _SO


def _load():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
        _lib.naju_oracle_threads.restype = ctypes.c_int
        for sfx in ("f32", "f64"):
            getattr(_lib, f"naju_oracle_bwd_{sfx}").restype = ctypes.c_int
            getattr(_lib, f"naju_oracle_fwd_{sfx}").restype = None
            getattr(_lib, f"naju_oracle_step_{sfx}").restype = None
    return _lib


def oracle_threads():
    return int(_load().naju_oracle_threads())


def _f32(a):
    if a is None:
        return None
    if hasattr(a, "detach"):
        a = a.detach().float().cpu().numpy()
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def oracle_fwd(u, fl, il, Bm, Cm, Dskip, h0=None, return_final_state=False, precision="f64"):
    u, fl, il, Bm, Cm, Dskip, h0 = map(_f32, (u, fl, il, Bm, Cm, Dskip, h0))
    B, T, D = u.shape
    N = Bm.shape[-1]
    assert N <= 128
    y = np.empty((B, T, D), np.float32)
    hT = np.empty((B, D, N), np.float32) if return_final_state else None
    getattr(_load(), f"naju_oracle_fwd_{precision}")(
        _p(u), _p(fl), _p(il), _p(Bm), _p(Cm), _p(Dskip), _p(h0), _p(y), _p(hT),
        ctypes.c_int(B), ctypes.c_int(T), ctypes.c_int(D), ctypes.c_int(N))
    return (y, hT) if return_final_state else y


def oracle_bwd(u, fl, il, Bm, Cm, Dskip, dy, h0=None, dhT=None, precision="f64"):
    """Returns dict(du, dfl, dil, dB, dC, dD, dh0)."""
    u, fl, il, Bm, Cm, Dskip, dy, h0, dhT = map(_f32, (u, fl, il, Bm, Cm, Dskip, dy, h0, dhT))
    B, T, D = u.shape
    N = Bm.shape[-1]
    assert N <= 128
    out = dict(du=np.empty_like(u), dfl=np.empty_like(u), dil=np.empty_like(u),
               dB=np.empty_like(Bm), dC=np.empty_like(Cm), dD=np.empty((D,), np.float32),
               dh0=np.empty((B, D, N), np.float32))
    rc = getattr(_load(), f"naju_oracle_bwd_{precision}")(
        _p(u), _p(fl), _p(il), _p(Bm), _p(Cm), _p(Dskip), _p(h0), _p(dy), _p(dhT),
        _p(out["du"]), _p(out["dfl"]), _p(out["dil"]), _p(out["dB"]), _p(out["dC"]),
        _p(out["dD"]), _p(out["dh0"]),
        ctypes.c_int(B), ctypes.c_int(T), ctypes.c_int(D), ctypes.c_int(N))
    if rc != 0:
        raise MemoryError("oracle backward could not allocate its scratch buffers")
    return out


def oracle_step(state, u, fl, il, Bm, Cm, Dskip, precision="f64"):
    """One decode step.  state [B,D,N]; u,fl,il [B,D]; Bm,Cm [B,N] -> (y [B,D], new state)."""
    state = _f32(state).copy()
    u, fl, il, Bm, Cm, Dskip = map(_f32, (u, fl, il, Bm, Cm, Dskip))
    B, D, N = state.shape
    y = np.empty((B, D), np.float32)
    getattr(_load(), f"naju_oracle_step_{precision}")(
        _p(state), _p(u), _p(fl), _p(il), _p(Bm), _p(Cm), _p(Dskip), _p(y),
        ctypes.c_int(B), ctypes.c_int(D), ctypes.c_int(N))
    return y, state


def make_inputs(B, T, D, N, seed=0, f_shift=2.0, i_shift=0.0, d_skip_scale=0.0,
                with_h0=False, bc_scale=None):
    """Seeded synthetic scan inputs with the distributions of the benchmark configs:
    u~N(0,1), f_logit~N(f_shift,1), i_logit~N(i_shift,1), B,C~N(0,bc_scale^2) with
    bc_scale = 1/sqrt(N) unless given, D_skip~N(0,d_skip_scale^2), dy~N(0,1).
    numpy's PCG64 stream (not torch's) so the values are the same on every machine."""
    g = np.random.default_rng(seed)
    r = lambda *s: g.standard_normal(s, dtype=np.float32)
    bc = np.float32(N ** -0.5 if bc_scale is None else bc_scale)
    d = dict(u=r(B, T, D), fl=r(B, T, D) + np.float32(f_shift), il=r(B, T, D) + np.float32(i_shift),
             Bm=r(B, T, N) * bc, Cm=r(B, T, N) * bc,
             Dskip=r(D) * np.float32(d_skip_scale), dy=r(B, T, D))
    d["h0"] = r(B, D, N) if with_h0 else None
    d["dhT"] = r(B, D, N) if with_h0 else None
    return d


def rel_l2(a, b):
    """||a-b|| / ||b|| over the whole tensor, in float64."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    den = np.linalg.norm(b.ravel())
    return float(np.linalg.norm((a - b).ravel()) / (den if den > 0 else 1.0))
