"""Failure reporting and framework composition of the scan on a GPU.

* A device-side wait that runs out must never yield silently wrong numbers: the call overwrites
  its own outputs with NaN on the device, and with NAJU_B200_CHECK_STATUS=1 the host layer also
  raises.  The failure is injected from the host (NAJU_FLAG_INJECT_TIMEOUT sets the status bit
  after the kernels; nothing on the GPU waits, traps or hangs).
* torch.utils.checkpoint(use_reentrant=False) around the scan (how NajuBlock(use_ckpt=True),
  naju/mixer.py:139-141, calls it) recomputes the forward during backward and must give the
  same gradients.
* torch.compile(fullgraph=True) of a function that calls naju_scan: the scan is a registered
  custom op with fake-tensor and autograd formulas, so there is no graph break
  (the reference's scan is one: naju/README.md:99-100).
"""
import numpy as np
import pytest
import torch
from torch.utils.checkpoint import checkpoint

import oracle

pytestmark = pytest.mark.gpu


def _leaves(B, T, D, N, seed, dtype=torch.float32):
    d = oracle.make_inputs(B, T, D, N, seed=seed, d_skip_scale=0.01)
    t = [torch.tensor(d[k], device="cuda").to(dtype if k != "Dskip" else torch.float32).requires_grad_(True)
         for k in ("u", "fl", "il", "Bm", "Cm", "Dskip")]
    return d, t


@pytest.mark.parametrize("shape,dtype", [((2, 300, 192, 16), torch.float32),       # recurrent kernels
                                         ((4, 300, 2432, 16), torch.bfloat16)])   # tcgen05 kernels
def test_injected_timeout_poisons_outputs_and_raises_when_checked(monkeypatch, shape, dtype):
    from naju_b200 import naju_scan
    B, T, D, N = shape
    d, t = _leaves(B, T, D, N, seed=31, dtype=dtype)
    monkeypatch.setenv("NAJU_B200_INJECT_TIMEOUT", "1")
    monkeypatch.setenv("NAJU_B200_CHECK_STATUS", "0")
    y, hT = naju_scan(*t, return_final_state=True)
    y.backward(torch.ones_like(y))
    torch.cuda.synchronize()
    assert bool(torch.isnan(y.float()).all()) and bool(torch.isnan(hT).all())
    for x in t:
        assert bool(torch.isnan(x.grad.float()).all())
    # with the status check on, the host layer raises instead of returning NaN
    monkeypatch.setenv("NAJU_B200_INJECT_TIMEOUT", "1")
    monkeypatch.setenv("NAJU_B200_CHECK_STATUS", "1")
    with pytest.raises(RuntimeError, match="bounded wait ran out"):
        naju_scan(*[x.detach() for x in t])
    # and a normal call afterwards is clean again
    monkeypatch.setenv("NAJU_B200_INJECT_TIMEOUT", "0")
    y = naju_scan(*[x.detach() for x in t])
    assert bool(torch.isfinite(y.float()).all())


def test_trailer_mark_of_a_failed_forward_reaches_the_backward(monkeypatch):
    """Through the C ABI: forward with the injection flag, backward WITHOUT it on the same
    checkpoints -> the backward's outputs are NaN because the forward marked the checkpoints."""
    from naju_b200 import _lib
    from naju_b200.scan import _desc, _prepare, scan_backward, scan_forward
    monkeypatch.setenv("NAJU_B200_CHECK_STATUS", "0")
    d, t = _leaves(1, 200, 128, 16, seed=32)
    p = _prepare(*[x.detach() for x in t])
    monkeypatch.setenv("NAJU_B200_INJECT_TIMEOUT", "1")
    y, _, _, ckpt, desc = scan_forward(*p)
    monkeypatch.setenv("NAJU_B200_INJECT_TIMEOUT", "0")
    clean = _desc(*p[:5])
    assert clean.flags & _lib.FLAG_INJECT_TIMEOUT == 0
    grads = scan_backward(clean, *p, None, torch.ones_like(y), None, ckpt)
    torch.cuda.synchronize()
    assert all(bool(torch.isnan(g.float()).all()) for g in grads[:6])


def test_activation_checkpointing_non_reentrant(monkeypatch):
    from naju_b200 import naju_scan
    monkeypatch.setenv("NAJU_B200_CHECK_STATUS", "1")
    d, t = _leaves(2, 260, 192, 16, seed=33)
    w = torch.randn(192, 192, device="cuda") * 0.05

    def block(u, fl, il, Bm, Cm, Dk):
        return naju_scan(u @ w, fl, il, Bm, Cm, Dk).tanh()

    dy = torch.tensor(d["dy"], device="cuda")
    block(*t).backward(dy)
    ref = [x.grad.clone() for x in t]
    for x in t:
        x.grad = None
    checkpoint(block, *t, use_reentrant=False).backward(dy)
    for x, r in zip(t, ref):
        assert oracle.rel_l2(x.grad.cpu().numpy(), r.cpu().numpy()) < 1e-5


@pytest.mark.parametrize("shape,dtype,state", [((2, 200, 192, 16), torch.float32, True),
                                               ((4, 300, 2432, 16), torch.bfloat16, False)])
def test_torch_compile_fullgraph_matches_eager(monkeypatch, shape, dtype, state):
    from naju_b200 import naju_scan
    monkeypatch.setenv("NAJU_B200_CHECK_STATUS", "1")
    B, T, D, N = shape
    d, t = _leaves(B, T, D, N, seed=34, dtype=dtype)
    h0 = torch.randn(B, D, N, device="cuda", requires_grad=True) if state else None

    def fn(u, fl, il, Bm, Cm, Dk, h):
        if h is None:
            return naju_scan(u * 1.0, fl, il, Bm, Cm, Dk).float().square().mean()
        y, hT = naju_scan(u * 1.0, fl, il, Bm, Cm, Dk, h0=h, return_final_state=True)
        return y.float().square().mean() + hT.square().mean()

    leaves = t + ([h0] if state else [])
    fn(*t, h0).backward()
    ref = [x.grad.clone() for x in leaves]
    ref_val = float(fn(*t, h0))
    for x in leaves:
        x.grad = None
    cfn = torch.compile(fn, fullgraph=True, backend="aot_eager")
    out = cfn(*t, h0)
    out.backward()
    assert abs(float(out) - ref_val) <= 1e-5 * abs(ref_val)
    for x, r in zip(leaves, ref):
        assert oracle.rel_l2(x.grad.float().cpu().numpy(), r.float().cpu().numpy()) < 1e-5


@pytest.mark.parametrize("shape", [(4, 520, 2440, 16, torch.bfloat16), (2, 1000, 200, 16, torch.bfloat16),
                                   (2, 300, 130, 24, torch.float32), (1, 65, 64, 100, torch.float32)])
def test_kernels_stay_inside_their_workspaces(monkeypatch, shape):
    """NAJU_B200_GUARD=1 puts canary bands around the checkpoint and scratch buffers of every call;
    after a forward and a backward in each kernel family (walk, ticket, recurrent; partial channel
    tiles, ragged T, wide states) the bands must be intact."""
    from naju_b200 import naju_scan
    from naju_b200 import scan as S
    monkeypatch.setenv("NAJU_B200_GUARD", "1")
    S.check_workspace_guards()
    B, T, D, N, dt = shape
    g = torch.Generator(device="cuda").manual_seed(3)
    r = lambda *s: torch.randn(*s, device="cuda", generator=g)
    u, fl, il = r(B, T, D).to(dt).requires_grad_(), (r(B, T, D) + 2).to(dt).requires_grad_(), r(B, T, D).to(dt).requires_grad_()
    Bm, Cm = (r(B, T, N) / N ** 0.5).to(dt).requires_grad_(), (r(B, T, N) / N ** 0.5).to(dt).requires_grad_()
    Dk = torch.zeros(D, device="cuda").requires_grad_()
    h0 = r(B, D, N).requires_grad_()
    y, hT = naju_scan(u, fl, il, Bm, Cm, Dk, h0=h0, return_final_state=True)
    torch.autograd.backward([y, hT], [r(B, T, D).to(dt), r(B, D, N)])
    torch.cuda.synchronize()
    assert S.check_workspace_guards() >= 3          # checkpoint + scratch (forward), scratch (backward)
    assert torch.isfinite(y.float()).all() and torch.isfinite(u.grad.float()).all()
