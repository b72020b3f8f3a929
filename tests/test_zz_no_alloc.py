"""The allocation-free forward entry point, naju_b200_fwd_noalloc.

It exists for callers that get only input and output buffers from their host runtime and may
not allocate device memory on that path (an inference engine's enqueue hook, a serving loop
that reserved all memory at start-up): the workspaces naju_b200_fwd() takes from the caller
come from a fixed array inside the library instead.  Checked here through the C ABI: two calls
in a row, which share that array and find the previous call's leftovers in it, must both match
the caller-workspace entry point; an oversized problem must be refused with a clear error.

This file is collected last on purpose, so that a run stopping at the first failure has
already run every other test.
"""
import ctypes

import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

# same bound the other fp32 GPU parity tests use (relative L2 over the whole tensor); the
# two entry points run the same kernel, only the look-back's folding order may differ
TIGHT_FWD = 2e-5


def _inputs(B, T, D, N, seed, dtype=torch.float32):
    d = oracle.make_inputs(B, T, D, N, seed=seed, d_skip_scale=0.01, with_h0=True)
    return {k: torch.tensor(d[k], device="cuda").to(torch.float32 if k in ("Dskip", "h0") else dtype)
            for k in ("u", "fl", "il", "Bm", "Cm", "Dskip", "h0")}


def _p(t):
    return None if t is None else t.data_ptr()


def _call_noalloc(lib, desc, t, y, hT):
    return lib.naju_b200_fwd_noalloc(desc, _p(t["u"]), _p(t["fl"]), _p(t["il"]), _p(t["Bm"]),
                                     _p(t["Cm"]), _p(t["Dskip"]), _p(t["h0"]), _p(y), _p(hT),
                                     torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("shapes", [[(2, 700, 200, 16, 1), (1, 333, 136, 24, 2)]])
def test_noalloc_forward_matches_caller_workspace_forward_twice(shapes):
    from naju_b200 import _lib
    from naju_b200.scan import _desc, scan_forward
    lib = _lib.load()
    for (B, T, D, N, seed) in shapes:      # second call reuses the array the first one dirtied
        t = _inputs(B, T, D, N, seed)
        y_ref, hT_ref, _, _, desc = scan_forward(t["u"], t["fl"], t["il"], t["Bm"], t["Cm"],
                                                 t["Dskip"], t["h0"], want_final=True)
        y = torch.full_like(y_ref, float("nan"))
        hT = torch.full_like(hT_ref, float("nan"))
        rc = _call_noalloc(lib, desc, t, y, hT)
        assert rc == 0, _lib.strerror(rc)
        torch.cuda.synchronize()
        stream = torch.cuda.current_stream().cuda_stream
        assert lib.naju_b200_noalloc_read_status(stream) == 0
        assert lib.naju_b200_noalloc_read_form(stream) == _lib.FORM_RECURRENT
        assert oracle.rel_l2(y.cpu().numpy(), y_ref.cpu().numpy()) < TIGHT_FWD
        assert oracle.rel_l2(hT.cpu().numpy(), hT_ref.cpu().numpy()) < TIGHT_FWD
        # and against the CPU oracle, so that both entry points being wrong together shows
        yo, hTo = oracle.oracle_fwd(*(t[k].cpu().numpy() for k in ("u", "fl", "il", "Bm", "Cm", "Dskip")),
                                    h0=t["h0"].cpu().numpy(), return_final_state=True)
        assert oracle.rel_l2(y.cpu().numpy(), yo) < TIGHT_FWD
        assert oracle.rel_l2(hT.cpu().numpy(), hTo) < TIGHT_FWD


def test_noalloc_forward_through_the_tensor_core_kernels_twice():
    """bf16 problems that take the TMA / tcgen05 kernels (first the ticket kernel with its
    look-back scratch, then the walk-along-time kernel), so that those run on the library's own
    workspace too: both must match the caller-workspace entry point bit for bit or to rounding,
    report a clean status word and the expected kernel family."""
    from naju_b200 import _lib
    from naju_b200.scan import scan_forward
    lib = _lib.load()
    bf = torch.bfloat16
    stream = torch.cuda.current_stream().cuda_stream
    for (B, T, D, N, seed, form) in [(2, 1000, 200, 16, 3, _lib.FORM_TC_TICKET),
                                     (4, 300, 1664, 16, 4, _lib.FORM_TC_WALK)]:
        t = _inputs(B, T, D, N, seed, dtype=bf)
        y_ref, hT_ref, _, _, desc = scan_forward(t["u"], t["fl"], t["il"], t["Bm"], t["Cm"],
                                                 t["Dskip"], t["h0"], want_final=True)
        y = torch.full_like(y_ref, float("nan"))
        hT = torch.full_like(hT_ref, float("nan"))
        rc = _call_noalloc(lib, desc, t, y, hT)
        assert rc == 0, _lib.strerror(rc)
        assert lib.naju_b200_noalloc_read_status(stream) == 0
        assert lib.naju_b200_noalloc_read_form(stream) == form
        # same kernel, same inputs: only the look-back's folding order may differ
        assert oracle.rel_l2(hT.cpu().numpy(), hT_ref.cpu().numpy()) < TIGHT_FWD
        assert oracle.rel_l2(y.float().cpu().numpy(), y_ref.float().cpu().numpy()) < 1e-3
        yo, hTo = oracle.oracle_fwd(*(t[k].float().cpu().numpy() for k in ("u", "fl", "il", "Bm", "Cm")),
                                    t["Dskip"].cpu().numpy(), h0=t["h0"].cpu().numpy(), return_final_state=True)
        assert oracle.rel_l2(hT.cpu().numpy(), hTo) < 1e-3
        assert oracle.rel_l2(y.float().cpu().numpy(), torch.tensor(yo).to(bf).float().numpy()) < 1e-3


def test_noalloc_rejects_problems_beyond_its_workspace():
    from naju_b200 import _lib
    lib = _lib.load()
    d = _lib.ScanDesc()
    d.B, d.T, d.D, d.N = 8, 16384, 2048, 16            # needs ~570 MB of workspace
    d.act_dtype = d.gate_dtype = d.bc_dtype = _lib.NAJU_BF16
    d.u_sb = d.fl_sb = d.il_sb = d.T * d.D
    d.u_st = d.fl_st = d.il_st = d.D
    d.bm_sb = d.cm_sb = d.T * d.N
    d.bm_st = d.cm_st = d.N
    assert lib.naju_b200_ckpt_bytes(d) + lib.naju_b200_fwd_scratch_bytes(d) > _lib.NOALLOC_BYTES
    rc = lib.naju_b200_fwd_noalloc(d, *([None] * 10))
    assert rc == _lib.E_TOO_LARGE
    assert "too large" in _lib.strerror(rc)
