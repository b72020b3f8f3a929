"""The benchmark configurations as GPU cases: the mixer-shaped call (config 1), the long near-1-retention
scan (config 2, reduced for the oracle; full size through size-independent properties), the
decode stack (config 3, one layer's update at full batch) and the wide-state config 4 (reduced).
"""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _status_checks(monkeypatch):
    monkeypatch.setenv("NAJU_B200_CHECK_STATUS", "1")


def _round(a, dtype):
    return torch.tensor(a).to(dtype).float().numpy()


@pytest.mark.parametrize("size", [(2, 300, 128, False), (4, 512, 1216, True)])
def test_config1_mixer_shaped_call_under_bf16_autocast(size):
    """Reproduces how naju/mixer.py:112-122 builds the six scan inputs (random weights, std 0.02,
    bf16 autocast): u is a transposed conv output (time-contiguous memory), B and C are two
    views of one [B,T,2N] tensor, the logits are fp32 next to bf16 activations.  The scan must
    take them as they come and match the oracle evaluated on exactly those values.  The second
    size is large enough for the walk-along-time tensor-core kernels (76 channel tiles, T a
    multiple of 8): there u must reach the kernels without a copy and the kernel forms are
    asserted."""
    from naju_b200 import naju_scan
    from naju_b200 import scan as S
    torch.manual_seed(1)
    Bsz, T, d_model, tensor_core = size
    N = 16
    d_inner = 2 * d_model
    dev = "cuda"
    W_in = torch.randn(2 * d_inner, d_model, device=dev) * 0.02
    conv_w = torch.randn(d_inner, 1, 4, device=dev) * 0.2
    conv_b = torch.zeros(d_inner, device=dev)
    W_x = torch.randn(2 * N, d_inner, device=dev) * 0.2
    W_f = torch.randn(d_inner, d_inner, device=dev) * 0.02
    W_i = torch.randn(d_inner, d_inner, device=dev) * 0.02
    f_bias = torch.full((d_inner,), 5.0, device=dev)
    i_bias = torch.full((d_inner,), -2.0, device=dev)
    hidden = torch.randn(Bsz, T, d_model, device=dev)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        x, z = F.linear(hidden, W_in).chunk(2, dim=-1)
        x = F.silu(F.conv1d(x.transpose(1, 2), conv_w, conv_b, padding=3, groups=d_inner)[..., :T].transpose(1, 2))
        Bm, Cm = torch.split(F.linear(x, W_x), [N, N], dim=-1)
        f_logit = F.linear(x, W_f) + f_bias
        i_logit = F.linear(x, W_i) + i_bias
    assert x.dtype == torch.bfloat16 and not x.is_contiguous() and x.stride(1) == 1
    assert f_logit.dtype == torch.float32 and Bm.stride(1) == 2 * N
    leaves = [t.detach().clone(memory_format=torch.preserve_format).requires_grad_(True)
              for t in (x, f_logit, i_logit)]
    bc = torch.cat([Bm, Cm], -1).detach().requires_grad_(True)
    Bv, Cv = torch.split(bc, [N, N], dim=-1)
    Dz = torch.zeros(d_inner, device=dev)
    y = naju_scan(leaves[0], leaves[1], leaves[2], Bv, Cv, Dz)
    assert y.dtype == torch.bfloat16 and y.shape == (Bsz, T, d_inner)
    dy = torch.randn_like(y)
    y.backward(dy)
    if tensor_core:
        torch.cuda.synchronize()
        assert S.last_kernel_forms() == {"fwd": 3, "bwd": 3}      # NAJU_FORM_TC_WALK
        pu = S._prepare(leaves[0].detach(), leaves[1].detach(), leaves[2].detach(), Bv.detach(), Cv.detach(), Dz)[0]
        assert pu.data_ptr() == leaves[0].data_ptr() and pu.stride(1) == 1      # taken as it came
        assert leaves[0].grad.stride() == leaves[0].stride()                    # and du in the same layout
    a = [t.detach().float().cpu().numpy() for t in (leaves[0], leaves[1], leaves[2], Bv, Cv, Dz)]
    yo = oracle.oracle_fwd(*a)
    g = oracle.oracle_bwd(*a, dy.float().cpu().numpy())
    bf = torch.bfloat16
    assert oracle.rel_l2(y.detach().float().cpu().numpy(), _round(yo, bf)) < 1e-3
    assert oracle.rel_l2(leaves[0].grad.float().cpu().numpy(), _round(g["du"], bf)) < 2e-3
    assert leaves[1].grad.dtype == torch.float32
    assert oracle.rel_l2(leaves[1].grad.cpu().numpy(), g["dfl"]) < 2e-3
    assert oracle.rel_l2(leaves[2].grad.cpu().numpy(), g["dil"]) < 2e-3
    dBC = bc.grad.float().cpu().numpy()
    assert oracle.rel_l2(dBC[..., :N], _round(g["dB"], bf)) < 2e-3
    assert oracle.rel_l2(dBC[..., N:], _round(g["dC"], bf)) < 2e-3


def test_config2_long_near_one_retention_reduced():
    """config 2's distribution (f_logit ~ N(4,1): horizons of hundreds of steps) at B=1, T=8192,
    D=128, bf16 I/O: stresses the carry across 128 chunks."""
    from naju_b200 import naju_scan
    B, T, D, N = 1, 8192, 128, 16
    d = oracle.make_inputs(B, T, D, N, seed=2, f_shift=4.0)
    bf = torch.bfloat16
    q = {k: _round(d[k], bf) for k in ("u", "fl", "il", "Bm", "Cm", "dy")}
    t = [torch.tensor(q[k], device="cuda").to(bf).requires_grad_(True) for k in ("u", "fl", "il", "Bm", "Cm")]
    Dz = torch.zeros(D, device="cuda")
    y, hT = naju_scan(*t, Dz, return_final_state=True)
    y.backward(torch.tensor(q["dy"], device="cuda").to(bf))
    a = (q["u"], q["fl"], q["il"], q["Bm"], q["Cm"], np.zeros(D, np.float32))
    yo, hTo = oracle.oracle_fwd(*a, return_final_state=True)
    g = oracle.oracle_bwd(*a, q["dy"])
    assert oracle.rel_l2(hT.detach().cpu().numpy(), hTo) < 1e-3
    assert oracle.rel_l2(y.detach().float().cpu().numpy(), _round(yo, bf)) < 1e-3
    for tt, k in zip(t, ("du", "dfl", "dil", "dB", "dC")):
        assert oracle.rel_l2(tt.grad.float().cpu().numpy(), _round(g[k], bf)) < 2e-3, k


def _metric_inputs(B, T, D, N, f_shift, seed, dtype=torch.bfloat16):
    g = torch.Generator(device="cuda").manual_seed(seed)
    r = lambda *s: torch.randn(*s, device="cuda", generator=g)
    return [r(B, T, D).to(dtype), (r(B, T, D) + f_shift).to(dtype), r(B, T, D).to(dtype),
            (r(B, T, N) / N ** 0.5).to(dtype), (r(B, T, N) / N ** 0.5).to(dtype)]


@pytest.mark.parametrize("cfg", [(8, 16384, 2048, 16, 2.0), (4, 65536, 2048, 16, 4.0)])
def test_full_size_properties(cfg):
    """At the benchmark's full sizes (metric config; config 2) the oracle is out of reach, so parity
    rests on properties that do not depend on size:
      composition  scanning [0,T) == scanning [0,s) then [s,T) from the carried state
                   (fp32 final state to 1e-5; bf16 y to the rounding-flip bound 1e-3)
      adjointness  y is linear in u, in B and in C for fixed gates, so with h0 = 0 and
                   D_skip = 0:  <dy,y> = <du,u> = <dB,B> = <dC,C>   (to 2e-3, with dy = y)."""
    from naju_b200 import naju_scan
    B, T, D, N, fs = cfg
    u, fl, il, Bm, Cm = _metric_inputs(B, T, D, N, fs, seed=0)
    Dz = torch.zeros(D, device="cuda")
    with torch.no_grad():
        y, hT = naju_scan(u, fl, il, Bm, Cm, Dz, return_final_state=True)
        s = T // 2 + 37
        y1, h1 = naju_scan(u[:, :s], fl[:, :s], il[:, :s], Bm[:, :s], Cm[:, :s], Dz, return_final_state=True)
        y2, h2 = naju_scan(u[:, s:], fl[:, s:], il[:, s:], Bm[:, s:], Cm[:, s:], Dz, h0=h1,
                           return_final_state=True)
        assert float((h2 - hT).norm() / hT.norm()) < 1e-5
        num = (y[:, :s].float() - y1.float()).pow(2).sum() + (y[:, s:].float() - y2.float()).pow(2).sum()
        assert float((num / y.float().pow(2).sum()).sqrt()) < 1e-3
        del y1, y2
    leaves = [t.requires_grad_(True) for t in (u, Bm, Cm)]
    y = naju_scan(leaves[0], fl, il, leaves[1], leaves[2], Dz)
    dy = y.detach().clone()          # a cotangent aligned with y, so <dy,y> = ||y||^2 is well away from 0
    y.backward(dy)
    dot = lambda a, b: float((a.double() * b.double()).sum())
    ref = dot(dy, y.detach())
    for t in leaves:
        assert abs(dot(t.grad, t.detach()) - ref) < 2e-3 * abs(ref)


def test_config3_decode_layer_update_full_batch():
    """One layer's state update of config 3 (batch 256, d_inner 2048, N 16, bf16 activations,
    fp32 state ~ N(0,1)); the 24-layer stack repeats this call with per-layer tensors."""
    from naju_b200 import naju_scan_step
    B, D, N = 256, 2048, 16
    d = oracle.make_inputs(B, 1, D, N, seed=3, with_h0=True)
    bf = torch.bfloat16
    q = {k: _round(d[k][:, 0], bf) for k in ("u", "fl", "il", "Bm", "Cm")}
    state = torch.tensor(d["h0"], device="cuda")
    y, st = naju_scan_step(state, *(torch.tensor(q[k], device="cuda").to(bf) for k in ("u", "fl", "il", "Bm", "Cm")),
                           torch.zeros(D, device="cuda"))
    yo, so = oracle.oracle_step(d["h0"], q["u"], q["fl"], q["il"], q["Bm"], q["Cm"], np.zeros(D, np.float32))
    assert oracle.rel_l2(st.cpu().numpy(), so) < 2e-5
    assert oracle.rel_l2(y.float().cpu().numpy(), _round(yo, bf)) < 1e-3


def test_config4_wide_state_reduced():
    """config 4's shape family (N=64, bf16) at a size the oracle finishes quickly."""
    from naju_b200 import naju_scan
    B, T, D, N = 2, 200, 256, 64
    d = oracle.make_inputs(B, T, D, N, seed=4)
    bf = torch.bfloat16
    q = {k: _round(d[k], bf) for k in ("u", "fl", "il", "Bm", "Cm", "dy")}
    t = [torch.tensor(q[k], device="cuda").to(bf).requires_grad_(True) for k in ("u", "fl", "il", "Bm", "Cm")]
    y = naju_scan(*t, torch.zeros(D, device="cuda"))
    y.backward(torch.tensor(q["dy"], device="cuda").to(bf))
    a = (q["u"], q["fl"], q["il"], q["Bm"], q["Cm"], np.zeros(D, np.float32))
    g = oracle.oracle_bwd(*a, q["dy"])
    assert oracle.rel_l2(y.detach().float().cpu().numpy(), _round(oracle.oracle_fwd(*a), bf)) < 1e-3
    for tt, k in zip(t, ("du", "dfl", "dil", "dB", "dC")):
        assert oracle.rel_l2(tt.grad.float().cpu().numpy(), _round(g[k], bf)) < 2e-3, k
