"""Generates the golden fixtures in this folder from the UNMODIFIED reference.

Run where the reference tree is mounted:

    python tests/golden/make_golden.py <path of the reference checkout>

Every fixture is produced by naju.scan.naju_scan_reference (naju/scan.py:79-93) and
torch autograd through it.  Inputs come from oracle.make_inputs (a seeded numpy
stream), so a fixture stores only the generator arguments, a checksum of the inputs
and the reference outputs.

The reference has no initial state, final state or decode step.  Those cases are
still produced by the unmodified reference function, by bracketing the sequence
with N neutral steps on each side:
  * N leading steps with f=1, i=1 (logits +40), B_t = e_k and u_t = h0[:, :, k] load an
    arbitrary h0 into the state exactly (sigmoid(40) == 1.0 in fp32);
  * N trailing steps with f=1, u=0 and C_t = e_k read the final state out as y.
Gradients w.r.t. the leading u give dh0; seeding the trailing y with dhT injects
the final-state adjoint.
"""
import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
if len(sys.argv) < 2:
    sys.exit("usage: make_golden.py <path of the reference checkout>")
REF = sys.argv[1]
sys.path.insert(0, REF)

from naju.scan import naju_scan_reference  # noqa: E402  (the reference itself)
from oracle import make_inputs  # noqa: E402

torch.set_num_threads(max(1, os.cpu_count() or 1))

# name -> (kwargs of make_inputs, post-processing tag)
CASES = {
    # config 0 of the reference's benchmark list
    "cfg0_B2_T512_D64_N16": dict(B=2, T=512, D=64, N=16, seed=0, f_shift=2.0, i_shift=0.0),
    # reference GPU smoke distribution (naju/tests/test_gpu_smoke.py:32-45)
    "smoke_B2_T256_D64_N16": dict(B=2, T=256, D=64, N=16, seed=10, f_shift=3.0, i_shift=-2.0,
                                  bc_scale=1.0, d_skip_scale=0.01),
    # ragged shapes of naju/tests/test_affine_chunk.py:84-86 (f+2, i-1, D_skip 0.01 N)
    "ragged_B1_T7_D32_N16": dict(B=1, T=7, D=32, N=16, seed=39, f_shift=2.0, i_shift=-1.0,
                                 d_skip_scale=0.01),
    "ragged_B2_T65_D64_N64": dict(B=2, T=65, D=64, N=64, seed=129, f_shift=2.0, i_shift=-1.0,
                                  d_skip_scale=0.01),
    "ragged_B1_T129_D96_N32": dict(B=1, T=129, D=96, N=32, seed=225, f_shift=2.0, i_shift=-1.0,
                                   d_skip_scale=0.01),
    "odd_B1_T33_D36_N24": dict(B=1, T=33, D=36, N=24, seed=5, f_shift=2.0, i_shift=-1.0,
                               d_skip_scale=0.01),
    "wide_B1_T64_D32_N128": dict(B=1, T=64, D=32, N=128, seed=6, f_shift=2.0, i_shift=-1.0,
                                 d_skip_scale=0.01),
    # deep gates (naju/tests/test_affine_chunk.py:101-115: f_logit - 14)
    "deep_B2_T128_D64_N64": dict(B=2, T=128, D=64, N=64, seed=7, f_shift=-12.0, i_shift=-1.0,
                                 d_skip_scale=0.01),
    # near-1 retention (the long-sequence config's distribution, short)
    "slow_B1_T300_D48_N16": dict(B=1, T=300, D=48, N=16, seed=2, f_shift=4.0, i_shift=0.0),
    # initial/final state extension, via neutral bracket steps
    "state_B2_T96_D32_N16": dict(B=2, T=96, D=32, N=16, seed=11, f_shift=2.0, i_shift=0.0,
                                 d_skip_scale=0.01, with_h0=True),
    # single-token decode step from a random state
    "step_B3_T1_D40_N16": dict(B=3, T=1, D=40, N=16, seed=12, f_shift=2.0, i_shift=0.0,
                               d_skip_scale=0.01, with_h0=True),
}


def checksum(d):
    h = hashlib.sha256()
    for k in ("u", "fl", "il", "Bm", "Cm", "Dskip", "dy", "h0", "dhT"):
        if d.get(k) is not None:
            h.update(np.ascontiguousarray(d[k]).tobytes())
    return h.hexdigest()


def run_plain(d):
    t = {k: torch.tensor(d[k], requires_grad=True) for k in ("u", "fl", "il", "Bm", "Cm", "Dskip")}
    y = naju_scan_reference(t["u"], t["fl"], t["il"], t["Bm"], t["Cm"], t["Dskip"])
    y.backward(torch.tensor(d["dy"]))
    out = dict(y=y.detach().numpy())
    for k, g in (("u", "du"), ("fl", "dfl"), ("il", "dil"), ("Bm", "dB"), ("Cm", "dC"), ("Dskip", "dD")):
        out[g] = t[k].grad.numpy()
    return out


def run_with_state(d):
    B, T, D = d["u"].shape
    N = d["Bm"].shape[-1]
    eye = torch.eye(N)
    big = 40.0
    t = {k: torch.tensor(d[k], requires_grad=True) for k in ("u", "fl", "il", "Bm", "Cm", "Dskip", "h0")}
    # leading N steps: u_t = h0[:, :, k], B_t = e_k, f = i = 1; y of those steps is ignored
    u_pre = t["h0"].permute(0, 2, 1)                         # [B, N, D]
    ones = torch.full((B, N, D), big)
    e = eye.unsqueeze(0).expand(B, N, N)
    zN = torch.zeros(B, N, N)
    # trailing N steps: f = 1, u = 0, C_t = e_k
    u_all = torch.cat([u_pre, t["u"], torch.zeros(B, N, D)], 1)
    fl_all = torch.cat([ones, t["fl"], ones], 1)
    il_all = torch.cat([ones, t["il"], -ones], 1)
    B_all = torch.cat([e, t["Bm"], zN], 1)
    C_all = torch.cat([zN, t["Cm"], e], 1)
    y_all = naju_scan_reference(u_all, fl_all, il_all, B_all, C_all, t["Dskip"])
    y = y_all[:, N:N + T]
    hT = y_all[:, N + T:].permute(0, 2, 1)                   # [B, D, N]
    # the y of the bracket steps is not part of the loss, so D_skip*u there adds no gradient
    loss = (y * torch.tensor(d["dy"])).sum() + (hT * torch.tensor(d["dhT"])).sum()
    loss.backward()
    out = dict(y=y.detach().numpy(), hT=hT.detach().numpy())
    for k, g in (("u", "du"), ("fl", "dfl"), ("il", "dil"), ("Bm", "dB"), ("Cm", "dC"),
                 ("Dskip", "dD"), ("h0", "dh0")):
        out[g] = t[k].grad.numpy()
    return out


def main():
    for name, kw in CASES.items():
        d = make_inputs(**kw)
        out = run_with_state(d) if kw.get("with_h0") else run_plain(d)
        meta = dict(kw)
        np.savez(os.path.join(HERE, name + ".npz"), __kwargs__=np.array(repr(meta)),
                 __sha256__=np.array(checksum(d)), **{k: v.astype(np.float32) for k, v in out.items()})
        print(name, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
