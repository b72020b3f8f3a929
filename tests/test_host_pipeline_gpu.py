"""The host-tensor pipeline (batch rows streamed through the GPU on three streams) against the
oracle, and against the plain device call on the same inputs."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def _round(a, dt):
    return torch.tensor(a).to(dt).float().numpy()


@pytest.mark.parametrize("rows,splits,T", [(1, 1, 200), (2, 1, 200), (5, 1, 200), (1, 3, 850), (1, 2, 600)])
def test_host_pipeline_matches_oracle(rows, splits, T):
    """bf16 I/O, 5 batch rows in chunks of 1 / 2 (ragged last chunk) / all at once, and rows cut
    into 3 / 2 time segments chained through the final state and its adjoint; outputs come back
    in pinned host tensors.  Same tolerances as the device path (1e-3 forward, 2e-3 gradients
    against the identically rounded fp64 oracle)."""
    from naju_b200 import scan_fwd_bwd_host
    B, D, N = 5, 256, 16
    dt = torch.bfloat16
    d = oracle.make_inputs(B, T, D, N, seed=11, d_skip_scale=0.05)
    q = {k: (_round(d[k], dt) if k in ("u", "fl", "il", "Bm", "Cm", "dy") else d[k]) for k in d}
    h = {k: torch.tensor(q[k]).to(dt).pin_memory() for k in ("u", "fl", "il", "Bm", "Cm", "dy")}
    out = scan_fwd_bwd_host(h["u"], h["fl"], h["il"], h["Bm"], h["Cm"], torch.tensor(q["Dskip"]), h["dy"],
                            rows_per_chunk=rows, time_splits=splits)
    torch.cuda.synchronize()
    a = (q["u"], q["fl"], q["il"], q["Bm"], q["Cm"], q["Dskip"])
    yo = oracle.oracle_fwd(*a)
    g = oracle.oracle_bwd(*a, q["dy"])
    assert not out["y"].is_cuda and out["y"].is_pinned()
    assert oracle.rel_l2(out["y"].float().numpy(), _round(yo, dt)) < 1e-3
    for k in ("du", "dfl", "dil", "dB", "dC"):
        assert oracle.rel_l2(out[k].float().numpy(), _round(g[k], dt)) < 2e-3, k
    assert oracle.rel_l2(out["dD"].numpy(), g["dD"]) < 1e-4


def test_host_pipeline_reuses_output_buffers_and_rejects_device_tensors():
    from naju_b200 import scan_fwd_bwd_host
    B, T, D, N = 3, 70, 128, 16
    d = oracle.make_inputs(B, T, D, N, seed=12)
    h = {k: torch.tensor(d[k]).pin_memory() for k in ("u", "fl", "il", "Bm", "Cm", "dy")}
    Dk = torch.tensor(d["Dskip"])
    out = scan_fwd_bwd_host(h["u"], h["fl"], h["il"], h["Bm"], h["Cm"], Dk, h["dy"])
    torch.cuda.synchronize()
    first = {k: v.clone() for k, v in out.items()}
    out2 = scan_fwd_bwd_host(h["u"], h["fl"], h["il"], h["Bm"], h["Cm"], Dk, h["dy"], out=out)
    torch.cuda.synchronize()
    assert out2 is out
    for k in first:
        assert oracle.rel_l2(out[k].numpy(), first[k].numpy()) < 2e-6, k
    yo = oracle.oracle_fwd(d["u"], d["fl"], d["il"], d["Bm"], d["Cm"], d["Dskip"])
    assert oracle.rel_l2(out["y"].numpy(), yo) < 2e-5
    with pytest.raises(ValueError):
        scan_fwd_bwd_host(h["u"].cuda(), h["fl"], h["il"], h["Bm"], h["Cm"], Dk, h["dy"])
