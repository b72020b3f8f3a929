"""CPU-side checks of the C ABI library: it loads, exports every symbol the header declares,
answers its size queries and rejects bad arguments — no kernel is launched here."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from naju_b200.build import build
    build()
    from naju_b200 import _lib
    return _lib.load()


def test_exports_every_declared_symbol(lib):
    from naju_b200 import _lib
    header = open(os.path.join(ROOT, "include", "naju_b200.h")).read()
    declared = set(re.findall(r"\b(naju_b200_[a-z0-9_]+)\s*\(", header))
    assert declared == set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name


def test_version_and_strerror(lib):
    from naju_b200 import _lib
    assert lib.naju_b200_version() == _lib.ABI_VERSION == 2
    assert lib.naju_b200_strerror(0) == b"ok"
    assert b"NULL" in lib.naju_b200_strerror(-1)


def _desc(B=8, T=16384, D=2048, N=16, dt=1):
    from naju_b200 import _lib
    d = _lib.ScanDesc()
    d.B, d.T, d.D, d.N = B, T, D, N
    d.act_dtype = d.gate_dtype = d.bc_dtype = dt
    d.u_sb = d.fl_sb = d.il_sb = T * D
    d.u_st = d.fl_st = d.il_st = D
    d.bm_sb = d.cm_sb = T * N
    d.bm_st = d.cm_st = N
    return d


def test_size_queries(lib):
    d = _desc()
    tc = lib.naju_b200_chunk_len(d)
    assert tc in (32, 64, 128, 256)
    nchunks = (d.T + tc - 1) // tc
    # chunk-end states [chunks][B][D][N] fp32 plus one decay product per channel and chunk
    assert lib.naju_b200_ckpt_bytes(d) >= nchunks * d.B * d.D * (d.N + 1) * 4
    assert lib.naju_b200_fwd_scratch_bytes(d) > 0
    assert lib.naju_b200_bwd_scratch_bytes(d) > 0
    assert lib.naju_b200_ckpt_bytes(_desc(N=0)) == 0
    assert lib.naju_b200_ckpt_bytes(_desc(N=129)) == 0


def test_argument_validation_without_launch(lib):
    # every rejection below happens before any CUDA call
    d = _desc(N=200)
    assert lib.naju_b200_fwd(d, *([None] * 13)) == -2
    d = _desc()
    d.gate_dtype = 2  # fp16 gates with bf16 activations
    assert lib.naju_b200_fwd(d, *([None] * 13)) == -3
    d = _desc()
    assert lib.naju_b200_fwd(d, *([None] * 13)) == -1
    assert lib.naju_b200_bwd(d, *([None] * 19)) == -1
    assert lib.naju_b200_step(d, *([None] * 9)) == -1
    assert lib.naju_b200_read_status(None, None) == -1


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from naju_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()


def test_cpu_tensors_are_rejected():
    import torch
    from naju_b200 import naju_scan, naju_scan_step, resolve_backend
    z, zn = torch.zeros(1, 4, 8), torch.zeros(1, 4, 16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        naju_scan(z, z, z, zn, zn, torch.zeros(8))
    with pytest.raises(RuntimeError):
        naju_scan_step(torch.zeros(1, 8, 16), z[:, 0], z[:, 0], z[:, 0], zn[:, 0], zn[:, 0], torch.zeros(8))
    with pytest.raises(ValueError):
        resolve_backend("nope")
    assert resolve_backend(None) == "b200" and resolve_backend("chunk") == "b200"


def test_descriptor_of_a_time_contiguous_u():
    """Host logic without a GPU: which layouts of u go to the kernels as they are, what the
    descriptor says about them, and what the library's stride check accepts."""
    import torch
    from naju_b200 import scan as S
    B, T, D, N = 2, 64, 40, 16
    u_bdt = torch.zeros(B, D, T, dtype=torch.bfloat16)
    u = u_bdt.transpose(1, 2)                      # [B,T,D] view of [B,D,T] memory
    assert S._time_contig(u)
    assert not S._time_contig(torch.zeros(B, T, D, dtype=torch.bfloat16))                      # ordinary layout
    assert not S._time_contig(torch.zeros(B, D, 60, dtype=torch.bfloat16).transpose(1, 2))     # T % 8 != 0 (16-bit)
    assert S._time_contig(torch.zeros(B, D, 60).transpose(1, 2))                               # fp32: T % 4 == 0
    assert not S._time_contig(torch.zeros(B, D, 1, dtype=torch.bfloat16).transpose(1, 2))      # T = 1: ambiguous
    z = torch.zeros(B, T, D, dtype=torch.bfloat16)
    zn = torch.zeros(B, T, N, dtype=torch.bfloat16)
    d = S._desc(u, z, z, zn, zn)
    assert (d.u_sb, d.u_st, d.u_sd) == (D * T, 1, T)
    d0 = S._desc(z, z, z, zn, zn)
    assert (d0.u_sb, d0.u_st, d0.u_sd) == (T * D, D, 1)


def test_stride_check_of_the_time_contiguous_layout(lib):
    # (every rejection below happens before any CUDA call: all pointers are NULL, so an accepted
    # descriptor ends at the NULL-pointer check, code -1, and a bad stride at -4)
    d = _desc()
    d.u_st, d.u_sd = 1, d.T                   # time-contiguous u: legal
    assert lib.naju_b200_fwd(d, *([None] * 13)) == -1
    d.u_sd = d.T - 1                          # channels overlap
    assert lib.naju_b200_fwd(d, *([None] * 13)) in (-1, -4)
    d = _desc()
    d.u_st = 1                                # channel-contiguous u cannot have a time stride of 1
    assert lib.naju_b200_fwd(d, *([None] * 13)) in (-1, -4)
