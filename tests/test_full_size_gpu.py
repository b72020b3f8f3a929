"""The benchmark's own configurations at full size against the CPU oracle.

The headline numbers are quoted on B=8, T=16384, D=2048, N=16 (bf16 I/O); here the tensor-core
kernels' outputs at exactly that size -- 256 chunks walked per channel tile -- are compared with
the oracle (fp32 flavour, all host threads, a few seconds) on the same bf16-quantised inputs:
y and all six gradients.  The same for the long-sequence configuration's distribution
(f_logit ~ N(4,1)) at B=4, T=32768 (512 chunks per tile), and for the wide-state configuration's
per-GPU shape (B=8, T=8192, D=4096, N=64) on a random subset of channels (channels are
independent given B and C, so the oracle can run on the subset alone; dB/dC, which sum over all
channels, are checked at reduced size elsewhere).

bf16 outputs are compared with the identically rounded oracle; tolerances are the build target:
1e-3 forward, 2e-3 gradients (relative L2 over the whole tensor).
"""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

TOL_FWD, TOL_GRAD = 1e-3, 2e-3
WALK, RECURRENT = 3, 1


@pytest.fixture(autouse=True)
def _status_checks(monkeypatch):
    monkeypatch.setenv("NAJU_B200_CHECK_STATUS", "1")


def _rel_l2(got, ref):
    """||got - ref|| / ||ref|| for torch CPU tensors of any float dtype, accumulated in fp64
    slice by slice (the tensors are GiB-sized)."""
    num = den = 0.0
    g, r = got.reshape(-1), ref.reshape(-1)
    step = 1 << 26
    for i in range(0, g.numel(), step):
        a, b = g[i:i + step].double(), r[i:i + step].double()
        num += float((a - b).pow(2).sum())
        den += float(b.pow(2).sum())
    return (num / den) ** 0.5 if den > 0 else num ** 0.5


def _inputs(B, T, D, N, f_shift, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    r = lambda *s: torch.randn(*s, device="cuda", generator=g)
    bf = torch.bfloat16
    return dict(u=r(B, T, D).to(bf), fl=(r(B, T, D) + f_shift).to(bf), il=r(B, T, D).to(bf),
                Bm=(r(B, T, N) / N ** 0.5).to(bf), Cm=(r(B, T, N) / N ** 0.5).to(bf), dy=r(B, T, D).to(bf))


def _as_bf16_rounded(a):
    return torch.from_numpy(a).to(torch.bfloat16)


@pytest.mark.parametrize("cfg", [(8, 16384, 2048, 16, 2.0, 0), (4, 32768, 2048, 16, 4.0, 2)],
                         ids=["metric_B8_T16384_D2048", "long_B4_T32768_D2048_near_one_retention"])
def test_tensor_core_kernels_at_full_size_match_oracle(cfg):
    from naju_b200 import naju_scan
    from naju_b200.scan import last_kernel_forms
    B, T, D, N, fs, seed = cfg
    t = _inputs(B, T, D, N, fs, seed)
    leaves = {k: t[k].requires_grad_(True) for k in ("u", "fl", "il", "Bm", "Cm")}
    Dz = torch.zeros(D, device="cuda", requires_grad=True)
    y, hT = naju_scan(leaves["u"], leaves["fl"], leaves["il"], leaves["Bm"], leaves["Cm"], Dz,
                      return_final_state=True)
    y.backward(t["dy"])
    torch.cuda.synchronize()
    assert last_kernel_forms() == {"fwd": WALK, "bwd": WALK}
    got = {"y": y.detach().cpu(), "hT": hT.detach().cpu(), "dD": Dz.grad.cpu()}
    for k, g in (("u", "du"), ("fl", "dfl"), ("il", "dil"), ("Bm", "dB"), ("Cm", "dC")):
        got[g] = leaves[k].grad.cpu()
    host = {k: t[k].detach().float().cpu().numpy() for k in ("u", "fl", "il", "Bm", "Cm", "dy")}
    del t, leaves, y, hT
    torch.cuda.empty_cache()
    a = (host["u"], host["fl"], host["il"], host["Bm"], host["Cm"], np.zeros(D, np.float32))
    yo, hTo = oracle.oracle_fwd(*a, return_final_state=True, precision="f32")
    assert _rel_l2(got["hT"], torch.from_numpy(hTo)) < TOL_FWD
    assert _rel_l2(got["y"], _as_bf16_rounded(yo)) < TOL_FWD
    del yo
    g = oracle.oracle_bwd(*a, host["dy"], precision="f32")
    for k in ("du", "dfl", "dil", "dB", "dC"):
        assert _rel_l2(got[k], _as_bf16_rounded(g[k])) < TOL_GRAD, k
    assert _rel_l2(got["dD"], torch.from_numpy(g["dD"])) < TOL_GRAD


def test_wide_state_per_gpu_shape_on_a_channel_subset():
    """B=8, T=8192, D=4096, N=64 (one GPU's share of the wide-state configuration): y, du,
    d f_logit, d i_logit on 256 randomly chosen channels against the oracle run on those
    channels alone."""
    from naju_b200 import naju_scan
    B, T, D, N = 8, 8192, 4096, 64
    t = _inputs(B, T, D, N, 2.0, 4)
    leaves = {k: t[k].requires_grad_(True) for k in ("u", "fl", "il", "Bm", "Cm")}
    Dz = torch.zeros(D, device="cuda")
    y = naju_scan(leaves["u"], leaves["fl"], leaves["il"], leaves["Bm"], leaves["Cm"], Dz)
    y.backward(t["dy"])
    torch.cuda.synchronize()
    sel = torch.randperm(D, generator=torch.Generator().manual_seed(4))[:256].sort().values.cuda()
    pick = lambda x: x.detach().index_select(2, sel).float().cpu()
    got = {"y": pick(y), "du": pick(leaves["u"].grad), "dfl": pick(leaves["fl"].grad), "dil": pick(leaves["il"].grad)}
    sub = {k: pick(t[k]).numpy() for k in ("u", "fl", "il", "dy")}
    Bm, Cm = t["Bm"].detach().float().cpu().numpy(), t["Cm"].detach().float().cpu().numpy()
    a = (sub["u"], sub["fl"], sub["il"], Bm, Cm, np.zeros(256, np.float32))
    yo = oracle.oracle_fwd(*a, precision="f32")
    assert _rel_l2(got["y"], _as_bf16_rounded(yo).float()) < TOL_FWD
    g = oracle.oracle_bwd(*a, sub["dy"], precision="f32")
    for k in ("du", "dfl", "dil"):
        assert _rel_l2(got[k], _as_bf16_rounded(g[k]).float()) < TOL_GRAD, k
