"""GPU parity: the CUDA scan (through the Python host layer and the C ABI) against the
reference's golden fixtures and the CPU oracle.

Tolerances (relative L2 over the whole tensor, from the build target): forward output and
final state 1e-3, gradients 2e-3.  The fp32 path is additionally held to a much tighter
regression bound, because it computes the same recurrence in the same precision.
"""
import os

import numpy as np
import pytest
import torch

import oracle
from conftest import golden_names, load_golden

pytestmark = pytest.mark.gpu

TOL_FWD, TOL_GRAD = 1e-3, 2e-3          # build target
TIGHT_FWD, TIGHT_GRAD = 2e-5, 1e-4      # fp32 regression bound
GRADS = (("du", "u"), ("dfl", "fl"), ("dil", "il"), ("dB", "Bm"), ("dC", "Cm"), ("dD", "Dskip"))


@pytest.fixture(autouse=True)
def _status_checks(monkeypatch):
    monkeypatch.setenv("NAJU_B200_CHECK_STATUS", "1")


def _dev(d, dtype=torch.float32, gate_dtype=None, grad=True):
    t = {}
    for k in ("u", "fl", "il", "Bm", "Cm", "Dskip", "h0"):
        if d.get(k) is None:
            t[k] = None
            continue
        dt = torch.float32 if k in ("Dskip", "h0") else (gate_dtype or dtype) if k in ("fl", "il") else dtype
        t[k] = torch.tensor(d[k], device="cuda").to(dt).requires_grad_(grad)
    return t


def _run(d, dtype=torch.float32, gate_dtype=None, state=False):
    from naju_b200 import naju_scan
    t = _dev(d, dtype, gate_dtype)
    if state:
        y, hT = naju_scan(t["u"], t["fl"], t["il"], t["Bm"], t["Cm"], t["Dskip"], h0=t["h0"],
                          return_final_state=True)
        dhT = torch.tensor(d["dhT"], device="cuda")
        torch.autograd.backward([y, hT], [torch.tensor(d["dy"], device="cuda").to(dtype), dhT])
    else:
        y = naju_scan(t["u"], t["fl"], t["il"], t["Bm"], t["Cm"], t["Dskip"])
        hT = None
        y.backward(torch.tensor(d["dy"], device="cuda").to(dtype))
    torch.cuda.synchronize()
    out = dict(y=y.detach().float().cpu().numpy())
    if hT is not None:
        out["hT"] = hT.detach().cpu().numpy()
        out["dh0"] = t["h0"].grad.float().cpu().numpy()
    for g, k in GRADS:
        out[g] = t[k].grad.float().cpu().numpy()
    return out


@pytest.mark.parametrize("name", golden_names())
def test_fp32_matches_reference_fixture(name):
    d, ref = load_golden(name)
    out = _run(d, state="hT" in ref)
    assert oracle.rel_l2(out["y"], ref["y"]) < TIGHT_FWD
    if "hT" in ref:
        assert oracle.rel_l2(out["hT"], ref["hT"]) < TIGHT_FWD
        assert oracle.rel_l2(out["dh0"], ref["dh0"]) < TIGHT_GRAD
    for g, _ in GRADS:
        assert oracle.rel_l2(out[g], ref[g]) < TIGHT_GRAD, g


SHAPES = [  # (B, T, D, N, f_shift) — multi-chunk, multi-channel-tile, ragged in T and D
    (2, 1000, 384, 16, 2.0),
    (1, 257, 200, 16, 4.0),
    (3, 130, 136, 32, 2.0),
    (1, 100, 260, 64, 2.0),
    (1, 70, 72, 100, 2.0),
    (1, 1, 8, 16, 2.0),
]


@pytest.mark.parametrize("shape", SHAPES)
def test_fp32_matches_oracle(shape):
    B, T, D, N, fs = shape
    d = oracle.make_inputs(B, T, D, N, seed=T + D, f_shift=fs, d_skip_scale=0.01, with_h0=True)
    out = _run(d, state=True)
    a = (d["u"], d["fl"], d["il"], d["Bm"], d["Cm"], d["Dskip"])
    y, hT = oracle.oracle_fwd(*a, h0=d["h0"], return_final_state=True)
    g = oracle.oracle_bwd(*a, d["dy"], h0=d["h0"], dhT=d["dhT"])
    assert oracle.rel_l2(out["y"], y) < TIGHT_FWD
    assert oracle.rel_l2(out["hT"], hT) < TIGHT_FWD
    assert oracle.rel_l2(out["dh0"], g["dh0"]) < TIGHT_GRAD
    for k, _ in GRADS:
        assert oracle.rel_l2(out[k], g[k]) < TIGHT_GRAD, k


def _round(a, dtype):
    return torch.tensor(a).to(dtype).float().numpy()


@pytest.mark.parametrize("dtype,gate_dtype", [(torch.bfloat16, None), (torch.bfloat16, torch.float32),
                                               (torch.float16, None)])
def test_low_precision_io_matches_identically_rounded_oracle(dtype, gate_dtype):
    """Inputs are quantised once; the oracle runs in fp64 on the same quantised values and its
    outputs are rounded the same way the kernel rounds them (the comparison
    naju/tests/test_affine_chunk.py:142-169 makes for bf16 I/O)."""
    B, T, D, N = 2, 300, 256, 16
    d = oracle.make_inputs(B, T, D, N, seed=5, d_skip_scale=0.01)
    q = dict(d)
    for k in ("u", "Bm", "Cm", "dy"):
        q[k] = _round(d[k], dtype)
    for k in ("fl", "il"):
        q[k] = _round(d[k], gate_dtype or dtype)
    out = _run(q, dtype, gate_dtype)
    a = (q["u"], q["fl"], q["il"], q["Bm"], q["Cm"], q["Dskip"])
    y = oracle.oracle_fwd(*a)
    g = oracle.oracle_bwd(*a, q["dy"])
    assert oracle.rel_l2(out["y"], _round(y, dtype)) < TOL_FWD
    for k, src in GRADS:
        gd = torch.float32 if k == "dD" else (gate_dtype or dtype) if k in ("dfl", "dil") else dtype
        assert oracle.rel_l2(out[k], _round(g[k], gd)) < TOL_GRAD, k


def _forms():
    from naju_b200.scan import last_kernel_forms
    return last_kernel_forms()


TICKET, WALK, RECURRENT = 2, 3, 1   # NAJU_FORM_* of include/naju_b200.h


@pytest.mark.parametrize("shape", [(2, 64, 128, 16, 2.0, TICKET), (2, 1000, 384, 16, 2.0, TICKET),
                                   (1, 300, 256, 16, -3.0, TICKET), (1, 300, 256, 16, -12.0, TICKET),
                                   # a partial channel tile (D % 128 = 72) in the ticket kernel
                                   (2, 1000, 200, 16, 2.0, TICKET),
                                   # enough channel tiles for the walk-along-time mode (ragged T)
                                   (4, 520, 2432, 16, 2.0, WALK), (4, 520, 2432, 16, -2.5, WALK),
                                   # ... with a partial last channel tile (D % 128 = 8)
                                   (4, 520, 2440, 16, 2.0, WALK)])
def test_tensor_core_chunked_forward(monkeypatch, shape):
    """The tcgen05 chunked form against the fp64 oracle on the same bf16-quantised inputs.
    NAJU_B200_FORM=chunked makes the call fail rather than fall back, and the kernel family
    that ran is read back and asserted.  The arithmetic error is measured on the fp32 final
    state; y is emitted in bf16, so it is compared with the oracle rounded the same way (both
    to 1e-3, the build target; a perturbation e before rounding moves about e/ulp of the
    outputs by one bf16 ulp, i.e. ~sqrt(e * 2^-8), measured ~3.6e-4).  Deep-gate tiles
    (f_shift <= -2.5) take the exact per-tile path and must meet the tight bound."""
    from naju_b200 import naju_scan
    monkeypatch.setenv("NAJU_B200_FORM", "chunked")
    B, T, D, N, fs, form = shape
    dt = torch.bfloat16
    d = oracle.make_inputs(B, T, D, N, seed=3, f_shift=fs, d_skip_scale=0.01, with_h0=True)
    q = {k: (_round(d[k], dt) if k in ("u", "fl", "il", "Bm", "Cm") else d[k]) for k in d}
    t = {k: torch.tensor(q[k], device="cuda").to(dt if k in ("u", "fl", "il", "Bm", "Cm") else torch.float32)
         for k in ("u", "fl", "il", "Bm", "Cm", "Dskip", "h0")}
    with torch.no_grad():
        y, hT = naju_scan(t["u"], t["fl"], t["il"], t["Bm"], t["Cm"], t["Dskip"], h0=t["h0"],
                          return_final_state=True)
    yo, hTo = oracle.oracle_fwd(q["u"], q["fl"], q["il"], q["Bm"], q["Cm"], q["Dskip"], h0=q["h0"],
                                return_final_state=True)
    assert _forms()["fwd"] == form
    deep = fs <= -2.5
    assert oracle.rel_l2(hT.cpu().numpy(), hTo) < (TIGHT_FWD if deep else TOL_FWD)
    assert oracle.rel_l2(y.float().cpu().numpy(), _round(yo, dt)) < TOL_FWD


def test_chunked_form_refuses_what_it_cannot_take(monkeypatch):
    """NAJU_B200_FORM=chunked on a problem no tensor-core kernel takes (N = 12 is not one of
    its state widths) must raise, not fall back."""
    from naju_b200 import naju_scan
    monkeypatch.setenv("NAJU_B200_FORM", "chunked")
    z = torch.zeros(1, 70, 64, device="cuda", dtype=torch.bfloat16)
    zn = torch.zeros(1, 70, 12, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no tensor-core kernel"):
        naju_scan(z, z, z, zn, zn, torch.zeros(64, device="cuda"))


@pytest.mark.parametrize("case", [(4, 256, 2432, 16, 2.0, True), (4, 520, 2432, 16, 2.0, False),
                                  (4, 520, 2432, 16, 4.0, True), (4, 520, 2432, 16, -2.5, True),
                                  # a partial last channel tile (D % 128 = 8), with and without states
                                  (4, 520, 2440, 16, 2.0, True), (4, 300, 2440, 16, 2.0, False),
                                  # more channel tiles than SMs (some CTAs walk two of them), and
                                  # only a third of the SMs busy
                                  (2, 300, 12800, 16, 2.0, True), (1, 260, 6400, 16, 2.0, False)])
def test_tensor_core_chunked_backward(case):
    """Forward and backward in the tcgen05 chunked form (the shapes have enough channel tiles for
    the walk-along-time kernels; f_shift=-2.5 makes deep-gate tiles, which must route to the exact
    recurrent backward) against the fp64 oracle on the same bf16-quantised inputs.  bf16 outputs
    are compared with the identically rounded oracle (2e-3, the gradient tolerance of the build);
    the fp32 outputs dD and dh0 carry no output rounding and show the arithmetic error."""
    from naju_b200 import naju_scan
    B, T, D, N, fs, state = case
    dt = torch.bfloat16
    d = oracle.make_inputs(B, T, D, N, seed=3, f_shift=fs, d_skip_scale=0.01 if state else 0.0, with_h0=True)
    q = {k: (_round(d[k], dt) if k in ("u", "fl", "il", "Bm", "Cm", "dy") else d[k]) for k in d}
    t = {k: torch.tensor(q[k], device="cuda").to(dt if k in ("u", "fl", "il", "Bm", "Cm") else torch.float32).requires_grad_(True)
         for k in ("u", "fl", "il", "Bm", "Cm", "Dskip", "h0")}
    if state:
        y, hT = naju_scan(t["u"], t["fl"], t["il"], t["Bm"], t["Cm"], t["Dskip"], h0=t["h0"], return_final_state=True)
        torch.autograd.backward([y, hT], [torch.tensor(q["dy"], device="cuda").to(dt), torch.tensor(d["dhT"], device="cuda")])
    else:
        y = naju_scan(t["u"], t["fl"], t["il"], t["Bm"], t["Cm"], t["Dskip"])
        y.backward(torch.tensor(q["dy"], device="cuda").to(dt))
    torch.cuda.synchronize()
    # the walk-along-time forward ran; the tensor-core backward did the work unless the forward
    # met deep-gate tiles, in which case the exact recurrent backward must have
    assert _forms() == {"fwd": WALK, "bwd": RECURRENT if fs <= -2.5 else WALK}
    a = (q["u"], q["fl"], q["il"], q["Bm"], q["Cm"], q["Dskip"])
    g = oracle.oracle_bwd(*a, q["dy"], h0=q["h0"] if state else None, dhT=d["dhT"] if state else None)
    for k, src in GRADS:
        ref = g[k] if k == "dD" else _round(g[k], dt)
        assert oracle.rel_l2(t[src].grad.float().cpu().numpy(), ref) < TOL_GRAD, k
    assert oracle.rel_l2(t["Dskip"].grad.cpu().numpy(), g["dD"]) < 1e-4
    if state:
        assert oracle.rel_l2(t["h0"].grad.cpu().numpy(), g["dh0"]) < 1e-4


@pytest.mark.parametrize("case", [(4, 256, 2432, 16, 2.0, True), (4, 520, 2432, 16, 4.0, False),
                                  (4, 300, 2440, 16, 2.0, True)])
def test_tensor_core_fp32_logits(case):
    """The mixer's dtype mix under bf16 autocast (bf16 u, B, C; fp32 logits and logit gradients)
    through the tensor-core forward and backward: the logits are not quantised, their gradients
    come back in fp32 and carry no output rounding, so they show the arithmetic error (the 2e-3
    gradient tolerance of the build; measured ~1e-5)."""
    from naju_b200 import naju_scan
    B, T, D, N, fs, state = case
    dt = torch.bfloat16
    d = oracle.make_inputs(B, T, D, N, seed=5, f_shift=fs, d_skip_scale=0.01, with_h0=True)
    q = {k: (_round(d[k], dt) if k in ("u", "Bm", "Cm", "dy") else d[k]) for k in d}
    t = {k: torch.tensor(q[k], device="cuda").to(dt if k in ("u", "Bm", "Cm") else torch.float32).requires_grad_(True)
         for k in ("u", "fl", "il", "Bm", "Cm", "Dskip", "h0")}
    if state:
        y, hT = naju_scan(t["u"], t["fl"], t["il"], t["Bm"], t["Cm"], t["Dskip"], h0=t["h0"], return_final_state=True)
        torch.autograd.backward([y, hT], [torch.tensor(q["dy"], device="cuda").to(dt), torch.tensor(d["dhT"], device="cuda")])
    else:
        y = naju_scan(t["u"], t["fl"], t["il"], t["Bm"], t["Cm"], t["Dskip"])
        y.backward(torch.tensor(q["dy"], device="cuda").to(dt))
    torch.cuda.synchronize()
    assert t["fl"].grad.dtype == torch.float32 and t["il"].grad.dtype == torch.float32
    assert _forms() == {"fwd": WALK, "bwd": WALK}
    a = (q["u"], q["fl"], q["il"], q["Bm"], q["Cm"], q["Dskip"])
    yo = oracle.oracle_fwd(*a, h0=q["h0"] if state else None)
    assert oracle.rel_l2(y.detach().float().cpu().numpy(), _round(yo, dt)) < TOL_FWD
    g = oracle.oracle_bwd(*a, q["dy"], h0=q["h0"] if state else None, dhT=d["dhT"] if state else None)
    for k, src in GRADS:
        got = t[src].grad.float().cpu().numpy()
        if src in ("fl", "il"):
            assert oracle.rel_l2(got, g[k]) < 2e-4, k
        else:
            ref = g[k] if k == "dD" else _round(g[k], dt)
            assert oracle.rel_l2(got, ref) < TOL_GRAD, k


@pytest.mark.parametrize("gate32", [False, True])
def test_tensor_core_forward_fp16(gate32):
    """fp16 activations (with fp16 or fp32 logits) at a shape the walk-along-time tensor-core forward
    takes; B and C stay bf16 (the tensor-core operand type).  The backward of this mix is the
    recurrent one.  Compared with the fp64 oracle on the same quantised inputs."""
    from naju_b200 import naju_scan
    B, T, D, N = 4, 300, 2432, 16
    dt = torch.float16
    d = oracle.make_inputs(B, T, D, N, seed=7, f_shift=2.0, d_skip_scale=0.01, with_h0=True)
    q = dict(d)
    for k in ("u", "dy") + (() if gate32 else ("fl", "il")):
        q[k] = _round(d[k], dt)
    for k in ("Bm", "Cm"):
        q[k] = _round(d[k], torch.bfloat16)
    t = {"u": torch.tensor(q["u"], device="cuda").to(dt),
         "fl": torch.tensor(q["fl"], device="cuda").to(torch.float32 if gate32 else dt),
         "il": torch.tensor(q["il"], device="cuda").to(torch.float32 if gate32 else dt),
         "Bm": torch.tensor(q["Bm"], device="cuda").to(torch.bfloat16),
         "Cm": torch.tensor(q["Cm"], device="cuda").to(torch.bfloat16),
         "Dskip": torch.tensor(q["Dskip"], device="cuda"), "h0": torch.tensor(q["h0"], device="cuda")}
    for v in t.values():
        v.requires_grad_(True)
    y, hT = naju_scan(t["u"], t["fl"], t["il"], t["Bm"], t["Cm"], t["Dskip"], h0=t["h0"], return_final_state=True)
    torch.autograd.backward([y, hT], [torch.tensor(q["dy"], device="cuda").to(dt), torch.tensor(d["dhT"], device="cuda")])
    torch.cuda.synchronize()
    assert _forms() == {"fwd": WALK, "bwd": RECURRENT}
    a = (q["u"], q["fl"], q["il"], q["Bm"], q["Cm"], q["Dskip"])
    yo, hTo = oracle.oracle_fwd(*a, h0=q["h0"], return_final_state=True)
    assert oracle.rel_l2(hT.detach().cpu().numpy(), hTo) < TOL_FWD
    assert oracle.rel_l2(y.detach().float().cpu().numpy(), _round(yo, dt)) < TOL_FWD
    g = oracle.oracle_bwd(*a, q["dy"], h0=q["h0"], dhT=d["dhT"])
    assert oracle.rel_l2(t["u"].grad.float().cpu().numpy(), _round(g["du"], dt)) < TOL_GRAD
    assert oracle.rel_l2(t["fl"].grad.float().cpu().numpy(), g["dfl"] if gate32 else _round(g["dfl"], dt)) < TOL_GRAD
    assert oracle.rel_l2(t["Bm"].grad.float().cpu().numpy(), _round(g["dB"], torch.bfloat16)) < TOL_GRAD


def test_bf16_channel_count_tma_cannot_describe():
    """D = 2434 is not a multiple of 8, so the bf16 row stride is not a multiple of 16 bytes and no
    TMA descriptor exists for these tensors: the call must quietly take the kernels that do not
    need one (here the exact recurrent kernels), with the same results."""
    from naju_b200 import naju_scan
    B, T, D, N = 4, 300, 2434, 16
    dt = torch.bfloat16
    d = oracle.make_inputs(B, T, D, N, seed=13, f_shift=2.0)
    q = {k: (_round(d[k], dt) if k in ("u", "fl", "il", "Bm", "Cm", "dy") else d[k]) for k in d}
    t = {k: torch.tensor(q[k], device="cuda").to(dt if k != "Dskip" else torch.float32).requires_grad_(True)
         for k in ("u", "fl", "il", "Bm", "Cm", "Dskip")}
    y = naju_scan(t["u"], t["fl"], t["il"], t["Bm"], t["Cm"], t["Dskip"])
    y.backward(torch.tensor(q["dy"], device="cuda").to(dt))
    torch.cuda.synchronize()
    assert _forms() == {"fwd": RECURRENT, "bwd": RECURRENT}
    a = (q["u"], q["fl"], q["il"], q["Bm"], q["Cm"], q["Dskip"])
    assert oracle.rel_l2(y.detach().float().cpu().numpy(), _round(oracle.oracle_fwd(*a), dt)) < TOL_FWD
    g = oracle.oracle_bwd(*a, q["dy"])
    for k, src in GRADS:
        ref = g[k] if k == "dD" else _round(g[k], dt)
        assert oracle.rel_l2(t[src].grad.float().cpu().numpy(), ref) < TOL_GRAD, k


def test_strided_bc_views_and_no_grad():
    """B and C arrive as two views of one [B,T,2N] tensor (naju/mixer.py:116)."""
    from naju_b200 import naju_scan
    B, T, D, N = 2, 150, 64, 16
    d = oracle.make_inputs(B, T, D, N, seed=9)
    bc = torch.tensor(np.concatenate([d["Bm"], d["Cm"]], -1), device="cuda")
    Bm, Cm = torch.split(bc, [N, N], dim=-1)
    with torch.no_grad():
        y = naju_scan(torch.tensor(d["u"], device="cuda"), torch.tensor(d["fl"], device="cuda"),
                      torch.tensor(d["il"], device="cuda"), Bm, Cm, torch.tensor(d["Dskip"], device="cuda"))
    ref = oracle.oracle_fwd(d["u"], d["fl"], d["il"], d["Bm"], d["Cm"], d["Dskip"])
    assert oracle.rel_l2(y.cpu().numpy(), ref) < TIGHT_FWD


def test_transposed_u_layout():
    """u arrives time-contiguous ([B,D,T] memory) from the mixer's conv (naju/mixer.py:115)."""
    from naju_b200 import naju_scan
    B, T, D, N = 1, 90, 40, 16
    d = oracle.make_inputs(B, T, D, N, seed=13)
    u = torch.tensor(d["u"], device="cuda").transpose(1, 2).contiguous().transpose(1, 2)
    assert not u.is_contiguous()
    y = naju_scan(u, torch.tensor(d["fl"], device="cuda"), torch.tensor(d["il"], device="cuda"),
                  torch.tensor(d["Bm"], device="cuda"), torch.tensor(d["Cm"], device="cuda"),
                  torch.tensor(d["Dskip"], device="cuda"))
    ref = oracle.oracle_fwd(d["u"], d["fl"], d["il"], d["Bm"], d["Cm"], d["Dskip"])
    assert oracle.rel_l2(y.cpu().numpy(), ref) < TIGHT_FWD


def test_run_to_run_reproducibility():
    """A single chunk involves no cross-chunk carry and must repeat bit for bit.  Across
    chunks the decoupled look-back folds predecessor summaries in whatever order they become
    available, so repeated runs agree to fp32 rounding rather than bitwise."""
    d = oracle.make_inputs(2, 64, 256, 16, seed=21)
    a, b = _run(d), _run(d)
    for k in a:
        assert np.array_equal(a[k], b[k]), k
    d = oracle.make_inputs(2, 700, 256, 16, seed=22)
    a, b = _run(d), _run(d)
    for k in a:
        assert oracle.rel_l2(a[k], b[k]) < 2e-6, k


def test_empty_time_axis():
    from naju_b200 import naju_scan
    h0 = torch.randn(2, 8, 16, device="cuda")
    z = torch.zeros(2, 0, 8, device="cuda")
    zn = torch.zeros(2, 0, 16, device="cuda")
    y, hT = naju_scan(z, z, z, zn, zn, torch.zeros(8, device="cuda"), h0=h0, return_final_state=True)
    assert y.shape == (2, 0, 8) and torch.equal(hT, h0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("N", [16, 24, 64])
def test_decode_step(dtype, N):
    from naju_b200 import naju_scan_step
    B, D = 5, 200
    d = oracle.make_inputs(B, 1, D, N, seed=N, d_skip_scale=0.01, with_h0=True)
    q = {k: (_round(d[k][:, 0], dtype) if k in ("u", "fl", "il", "Bm", "Cm") else d[k]) for k in d}
    state = torch.tensor(d["h0"], device="cuda")
    y, st = naju_scan_step(state, *(torch.tensor(q[k], device="cuda").to(dtype) for k in ("u", "fl", "il", "Bm", "Cm")),
                           torch.tensor(d["Dskip"], device="cuda"))
    yo, so = oracle.oracle_step(d["h0"], q["u"], q["fl"], q["il"], q["Bm"], q["Cm"], d["Dskip"])
    assert st.data_ptr() == state.data_ptr()
    assert oracle.rel_l2(st.cpu().numpy(), so) < TIGHT_FWD
    assert oracle.rel_l2(y.float().cpu().numpy(), _round(yo, dtype)) < (TIGHT_FWD if dtype == torch.float32 else TOL_FWD)


def test_rejects_cpu_tensors_and_unknown_backend():
    from naju_b200 import naju_scan
    z = torch.zeros(1, 4, 8)
    zn = torch.zeros(1, 4, 16)
    with pytest.raises(RuntimeError):
        naju_scan(z, z, z, zn, zn, torch.zeros(8))
    with pytest.raises(ValueError):
        naju_scan(z, z, z, zn, zn, torch.zeros(8), backend="nope")


@pytest.mark.parametrize("case", [(4, 520, 2432, 8, 2.0, True), (4, 520, 2432, 12, 2.0, False),
                                  # deep gates: exact tiles forward, recurrent backward
                                  (4, 300, 2432, 8, -2.5, True)])
def test_fewer_than_16_states_take_the_tensor_core_form(case):
    """N < 16 on a problem large enough for the tcgen05 form: the host adds zero columns to B and
    C (and to h0 / dhT) up to the 16 states the kernels are built for, and slices the state-shaped
    results back.  Against the fp64 oracle at the original N on the same bf16-quantised inputs, at
    the build's tolerances; the kernel forms are asserted."""
    from naju_b200 import naju_scan
    B, T, D, N, fs, state = case
    dt = torch.bfloat16
    d = oracle.make_inputs(B, T, D, N, seed=5, f_shift=fs, d_skip_scale=0.01, with_h0=True)
    q = {k: (_round(d[k], dt) if k in ("u", "fl", "il", "Bm", "Cm", "dy") else d[k]) for k in d}
    t = {k: torch.tensor(q[k], device="cuda").to(dt if k in ("u", "fl", "il", "Bm", "Cm") else torch.float32).requires_grad_(True)
         for k in ("u", "fl", "il", "Bm", "Cm", "Dskip", "h0")}
    dy = torch.tensor(q["dy"], device="cuda").to(dt)
    if state:
        y, hT = naju_scan(t["u"], t["fl"], t["il"], t["Bm"], t["Cm"], t["Dskip"], h0=t["h0"], return_final_state=True)
        torch.autograd.backward([y, hT], [dy, torch.tensor(d["dhT"], device="cuda")])
    else:
        y = naju_scan(t["u"], t["fl"], t["il"], t["Bm"], t["Cm"], t["Dskip"])
        y.backward(dy)
    torch.cuda.synchronize()
    assert _forms() == {"fwd": WALK, "bwd": RECURRENT if fs <= -2.5 else WALK}
    a = (q["u"], q["fl"], q["il"], q["Bm"], q["Cm"], q["Dskip"])
    if state:
        yo, hTo = oracle.oracle_fwd(*a, h0=q["h0"], return_final_state=True)
        assert hT.shape == (B, D, N)
        assert oracle.rel_l2(hT.detach().cpu().numpy(), hTo) < TOL_FWD
    else:
        yo = oracle.oracle_fwd(*a)
    assert oracle.rel_l2(y.detach().float().cpu().numpy(), _round(yo, dt)) < TOL_FWD
    g = oracle.oracle_bwd(*a, q["dy"], h0=q["h0"] if state else None, dhT=d["dhT"] if state else None)
    for k, src in GRADS:
        ref = g[k] if k == "dD" else _round(g[k], dt)
        assert t[src].grad.shape == t[src].shape
        assert oracle.rel_l2(t[src].grad.float().cpu().numpy(), ref) < TOL_GRAD, k
    if state:
        assert oracle.rel_l2(t["h0"].grad.cpu().numpy(), g["dh0"]) < TOL_GRAD


@pytest.mark.parametrize("case", [
    # tensor-core walk kernels, forward and backward, D_skip and states
    (4, 520, 2432, 16, 2.0, torch.bfloat16, torch.bfloat16, WALK, WALK),
    # ... with fp32 logits (the mixer's dtypes) and a partial channel tile
    (4, 520, 2440, 16, 2.0, torch.bfloat16, torch.float32, WALK, WALK),
    # deep gates: exact tiles in the forward, recurrent backward (transposing tile loader)
    (4, 264, 2432, 16, -2.5, torch.bfloat16, torch.bfloat16, WALK, RECURRENT),
    # too few channel tiles for the walk: the ticket kernel does not take this layout, the
    # recurrent kernels do
    (2, 1000, 384, 16, 2.0, torch.bfloat16, torch.bfloat16, RECURRENT, RECURRENT),
    # fp32 everything (recurrent kernels)
    (2, 200, 300, 16, 2.0, torch.float32, torch.float32, RECURRENT, RECURRENT)])
def test_time_contiguous_u_is_taken_without_a_copy(case):
    """u as the mixer's depthwise convolution leaves it: [B,D,T] memory viewed as [B,T,D]
    (naju/mixer.py:115).  The host hands it to the kernels as it is (same data pointer, channel
    stride in the descriptor); the walk kernels read it through a (T, D, B) tensor map, the
    recurrent kernels transpose their tile while staging it.  Forward, final state and all
    gradients against the fp64 oracle on the same quantised inputs; kernel forms asserted."""
    from naju_b200 import naju_scan
    from naju_b200 import scan as S
    B, T, D, N, fs, dt, gdt, ffwd, fbwd = case
    d = oracle.make_inputs(B, T, D, N, seed=17, f_shift=fs, d_skip_scale=0.05, with_h0=True)
    cast = {"u": dt, "Bm": dt, "Cm": dt, "dy": dt, "fl": gdt, "il": gdt}
    q = {k: (_round(d[k], cast[k]) if k in cast else d[k]) for k in d}
    t = {k: torch.tensor(q[k], device="cuda").to(cast.get(k, torch.float32)) for k in ("u", "fl", "il", "Bm", "Cm", "Dskip", "h0")}
    t["u"] = t["u"].transpose(1, 2).contiguous().transpose(1, 2)      # [B,D,T] memory
    assert t["u"].stride() == (D * T, 1, T)
    for k in t:
        t[k].requires_grad_(True)
    pu = S._prepare(t["u"].detach(), t["fl"].detach(), t["il"].detach(), t["Bm"].detach(), t["Cm"].detach(),
                    t["Dskip"].detach())[0]
    assert pu.data_ptr() == t["u"].data_ptr() and pu.stride() == t["u"].stride()      # no copy
    y, hT = naju_scan(t["u"], t["fl"], t["il"], t["Bm"], t["Cm"], t["Dskip"], h0=t["h0"], return_final_state=True)
    torch.autograd.backward([y, hT], [torch.tensor(q["dy"], device="cuda").to(dt), torch.tensor(d["dhT"], device="cuda")])
    torch.cuda.synchronize()
    assert _forms() == {"fwd": ffwd, "bwd": fbwd}
    a = (q["u"], q["fl"], q["il"], q["Bm"], q["Cm"], q["Dskip"])
    yo, hTo = oracle.oracle_fwd(*a, h0=q["h0"], return_final_state=True)
    g = oracle.oracle_bwd(*a, q["dy"], h0=q["h0"], dhT=d["dhT"])
    f32 = dt == torch.float32
    tol_f, tol_g = (TIGHT_FWD, TIGHT_GRAD) if f32 else (TOL_FWD, TOL_GRAD)
    assert oracle.rel_l2(hT.detach().cpu().numpy(), hTo) < tol_f
    assert oracle.rel_l2(y.detach().float().cpu().numpy(), _round(yo, dt)) < tol_f
    for k, src in GRADS:
        gd = torch.float32 if k == "dD" else gdt if k in ("dfl", "dil") else dt
        assert t[src].grad.shape == t[src].shape
        assert oracle.rel_l2(t[src].grad.float().cpu().numpy(), _round(g[k], gd)) < tol_g, k
    assert oracle.rel_l2(t["h0"].grad.cpu().numpy(), g["dh0"]) < tol_g
