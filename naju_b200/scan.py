"""Host side of the B200 gated scan: the reference's scan interface over the C ABI.

Mirrors naju/scan.py of the reference project: the same `naju_scan` signature
(naju/scan.py:75-76), the same tensor meaning (naju/scan.py:3-12) and the same backend
selection rule (argument > NAJU_SCAN_BACKEND > default, naju/scan.py:48-52).  There is one
implementation behind it — hand-written sm_100a CUDA in libnaju_b200.so — and no fallback:
a CPU tensor or a missing library raises.

Additive, keyword-only extensions the reference does not have: an initial state `h0`, the
returned final state, and `naju_scan_step` for single-token decode.
"""
import os

import torch

from . import _lib

# The reference's backend names are accepted so that existing configs keep working
# (naju/mixer.py:121-122 forwards `scan_backend`); they all select the one CUDA path.
_ALIASES = ("b200", "reference", "chunk", "cuda", "cuda_bw", "affine", "fused_affine_chunk")

_DT = {torch.float32: _lib.NAJU_F32, torch.bfloat16: _lib.NAJU_BF16, torch.float16: _lib.NAJU_F16}


def resolve_backend(backend=None):
    """Same precedence as naju/scan.py:48-52; every valid name resolves to "b200"."""
    b = backend or os.environ.get("NAJU_SCAN_BACKEND") or "b200"
    b = b.lower()
    if b not in _ALIASES:
        raise ValueError(f"unknown scan backend {b!r}; valid: {', '.join(_ALIASES)}")
    return "b200"


def _form():
    """NAJU_B200_FORM selects the forward kernel family: "auto" (default) takes the tcgen05
    tensor-core chunked form where it applies (16-bit activations, bf16 B/C, N == 16 -- or fewer,
    padded with zero columns by the host when the problem is large enough --, TMA-legal strides) and the exact recurrent kernels elsewhere; "recurrent" forces the recurrent ones;
    "chunked" insists on the tensor-core form and raises where it does not apply."""
    f = os.environ.get("NAJU_B200_FORM", "auto").lower()
    if f not in ("auto", "chunked", "recurrent"):
        raise ValueError(f"NAJU_B200_FORM must be 'auto', 'chunked' or 'recurrent', got {f!r}")
    return f


def _check_status_enabled():
    return os.environ.get("NAJU_B200_CHECK_STATUS", "0") == "1"


# Kernel family (FORM_* of _lib) that did the work of the last forward / backward call, recorded
# when NAJU_B200_CHECK_STATUS=1 (reading it synchronises the stream).
_last_forms = {"fwd": None, "bwd": None}


def last_kernel_forms():
    """{"fwd": form, "bwd": form} of the most recent calls made with NAJU_B200_CHECK_STATUS=1."""
    return dict(_last_forms)


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _time_contig(u):
    """True for a [B,T,D] view of [B,D,T] memory (time stride 1, channels T or more apart) that
    the kernels can take as it is: what the mixer's depthwise convolution leaves behind
    (naju/mixer.py:115).  TMA wants the channel and batch strides to be multiples of 16 bytes."""
    if u.dim() != 3 or u.shape[1] < 2 or u.shape[2] < 2:
        return False
    sb, st, sd = u.stride()
    es = u.element_size()
    return (st == 1 and sd >= u.shape[1] and sb >= 0 and u.data_ptr() % 16 == 0 and
            (sd * es) % 16 == 0 and (sb * es) % 16 == 0 and (u.shape[0] == 1 or sb >= sd * u.shape[2]))


def _inner_contig(t):
    """Tensors whose last stride is 1 and whose outer strides are non-negative pass through."""
    if t.stride(-1) == 1 and all(s >= 0 for s in t.stride()) and t.data_ptr() % t.element_size() == 0:
        if t.dim() < 3 or t.stride(-2) >= t.shape[-1]:
            return t
    return t.contiguous()


def _prepare(u, f_logit, i_logit, Bm, Cm, D_skip):
    if not u.is_cuda:
        raise RuntimeError("naju_b200 scan needs CUDA tensors (there is no CPU fallback)")
    if u.dim() != 3 or f_logit.shape != u.shape or i_logit.shape != u.shape:
        raise ValueError("u, f_logit, i_logit must all be [B, T, D]")
    if Bm.dim() != 3 or Bm.shape != Cm.shape or Bm.shape[:2] != u.shape[:2]:
        raise ValueError("B and C must both be [B, T, N] matching u's batch and time")
    if D_skip.shape != (u.shape[-1],):
        raise ValueError("D_skip must be [D]")
    if Bm.shape[-1] < 1 or Bm.shape[-1] > 128:
        raise RuntimeError("d_state must be in 1..128")
    if u.dtype not in _DT:
        raise RuntimeError(f"unsupported dtype {u.dtype}")
    # gates run in u's dtype or fp32 (autocast hands fp32 logits next to bf16 activations)
    gdt = u.dtype if (f_logit.dtype == u.dtype and i_logit.dtype == u.dtype) else torch.float32
    f_logit = f_logit.to(gdt)
    i_logit = i_logit.to(gdt)
    bdt = Bm.dtype if (Bm.dtype == Cm.dtype and Bm.dtype in _DT) else torch.float32
    Bm, Cm = Bm.to(bdt), Cm.to(bdt)
    if not _time_contig(u):   # (a time-contiguous u goes to the kernels without a copy)
        u = _inner_contig(u)
    f_logit, i_logit, Bm, Cm = map(_inner_contig, (f_logit, i_logit, Bm, Cm))
    D_skip = D_skip.detach().to(torch.float32).contiguous()
    return u, f_logit, i_logit, Bm, Cm, D_skip


def _desc(u, f_logit, i_logit, Bm, Cm):
    B, T, D = u.shape
    d = _lib.ScanDesc()
    d.B, d.T, d.D, d.N = B, T, D, Bm.shape[-1]
    d.act_dtype, d.gate_dtype, d.bc_dtype = _DT[u.dtype], _DT[f_logit.dtype], _DT[Bm.dtype]
    form = _form()
    d.flags = (_lib.FLAG_RECURRENT_ONLY if form == "recurrent" else
               _lib.FLAG_CHUNKED_ONLY if form == "chunked" else 0)
    if os.environ.get("NAJU_B200_INJECT_TIMEOUT", "0") == "1":  # fault injection for tests
        d.flags |= _lib.FLAG_INJECT_TIMEOUT
    d.u_sb, d.u_st = u.stride(0), u.stride(1)
    d.u_sd = u.stride(2) if (u.stride(2) != 1 and u.stride(1) == 1) else 1
    d.fl_sb, d.fl_st = f_logit.stride(0), f_logit.stride(1)
    d.il_sb, d.il_st = i_logit.stride(0), i_logit.stride(1)
    d.bm_sb, d.bm_st = Bm.stride(0), Bm.stride(1)
    d.cm_sb, d.cm_st = Cm.stride(0), Cm.stride(1)
    if T <= 1:  # a size-1 dimension may carry any stride; give the kernel a legal one
        d.u_st, d.fl_st, d.il_st = max(d.u_st, D), max(d.fl_st, D), max(d.il_st, D)
        d.bm_st, d.cm_st = max(d.bm_st, d.N), max(d.cm_st, d.N)
    return d


_GUARD = 4096          # bytes of canary on each side of a workspace when NAJU_B200_GUARD=1
_GUARD_BYTE = 0xA5
_guarded = []          # (whole buffer, payload size) of the workspaces handed out since the last check


def _workspace(nbytes, device):
    """Caller-owned workspace for the library (torch's caching allocator returns 512-byte aligned
    blocks).  With NAJU_B200_GUARD=1 every workspace sits between two canary bands that
    check_workspace_guards() verifies: the stand-in for a memory checker on the kernels' writes to
    checkpoint and scratch buffers (a debug aid; off by default)."""
    n = max(int(nbytes), 256)
    if os.environ.get("NAJU_B200_GUARD", "0") != "1":
        return torch.empty(n, dtype=torch.uint8, device=device)
    n_al = (n + 255) // 256 * 256
    whole = torch.empty(_GUARD + n_al + _GUARD, dtype=torch.uint8, device=device)
    whole[:_GUARD] = _GUARD_BYTE
    whole[_GUARD + n:] = _GUARD_BYTE
    _guarded.append((whole, n))
    return whole[_GUARD:_GUARD + n]


def check_workspace_guards():
    """Verifies (and forgets) the canary bands of every workspace handed out under
    NAJU_B200_GUARD=1 since the last call; raises if a kernel wrote outside its workspace.
    Synchronises the device."""
    bad = []
    for whole, n in _guarded:
        lo, hi = whole[:_GUARD], whole[_GUARD + n:]
        if bool((lo != _GUARD_BYTE).any()) or bool((hi != _GUARD_BYTE).any()):
            bad.append((int(whole.numel()), n))
    count = len(_guarded)
    _guarded.clear()
    if bad:
        raise RuntimeError(f"workspace guard bands overwritten: {bad}")
    return count


def _state_arg(h, B, D, N, name):
    if h is None:
        return None
    if h.shape != (B, D, N):
        raise ValueError(f"{name} must be [B, D, N]")
    return h.detach().to(torch.float32).contiguous()


# ---------------------------------------------------------------------------------------------
# Fewer than 16 states.  The tcgen05 kernels are built for 16 states; the recurrence
# (naju/scan.py:87-91) is diagonal in the state index and y only sums over it, so zero columns
# added to B and C (and to h0 / dhT) change nothing: the host pads N < 16 up to 16 and slices the
# state-shaped results back.  (The same argument splits N > 16 into groups of 16 states whose
# y / du / d f_logit / d i_logit are added up; that was built and measured -- 2.2x (N=64) and 3.1x
# (N=32) faster than the recurrent kernels at B=8, T=8192, D=4096 -- but every group's output is
# rounded to the 16-bit activation type before the sum, which put y and the gradients at 2.7e-3 of
# the reference, outside the 1e-3 / 2e-3 bounds, so N > 16 stays with the exact recurrent kernels.)
_GROUP = 16
_PAD_MIN_WORK = 1 << 20  # B*T*D below which the recurrent kernels are as fast


def _pad_to_group(u, Bm):
    """True if B and C get zero columns up to 16 states so that the tensor-core form applies."""
    if Bm.shape[-1] >= _GROUP or _form() == "recurrent":
        return False
    if u.dtype not in (torch.bfloat16, torch.float16) or Bm.dtype != torch.bfloat16:
        return False
    B, T, D = u.shape
    return B * T * D >= _PAD_MIN_WORK and T >= 128


def _pad_states(t):
    """Zero columns up to 16 along the last dimension (a copy; these tensors are small)."""
    if t is None or t.shape[-1] == _GROUP:
        return t
    return torch.nn.functional.pad(t, (0, _GROUP - t.shape[-1]))


def scan_forward(u, f_logit, i_logit, Bm, Cm, D_skip, h0=None, want_final=False, want_decay=False):
    """Raw forward over prepared tensors.  Returns (y, hT|None, pT|None, ckpt, desc)."""
    lib = _lib.load()
    B, T, D = u.shape
    N = Bm.shape[-1]
    if _pad_to_group(u, Bm):
        Bm, Cm, h0 = _pad_states(Bm), _pad_states(Cm), _pad_states(h0)
    Np = Bm.shape[-1]
    d = _desc(u, f_logit, i_logit, Bm, Cm)
    dev = u.device
    y = torch.empty((B, T, D), dtype=u.dtype, device=dev)
    hT = torch.empty((B, D, Np), dtype=torch.float32, device=dev) if want_final else None
    pT = torch.empty((B, D), dtype=torch.float32, device=dev) if want_decay else None
    ckpt = _workspace(lib.naju_b200_ckpt_bytes(d), dev)
    scratch = _workspace(lib.naju_b200_fwd_scratch_bytes(d), dev)
    with torch.cuda.device(dev):
        rc = lib.naju_b200_fwd(d, _ptr(u), _ptr(f_logit), _ptr(i_logit), _ptr(Bm), _ptr(Cm),
                               _ptr(D_skip), _ptr(h0), _ptr(y), _ptr(hT), _ptr(pT), _ptr(ckpt),
                               _ptr(scratch), _stream())
        _lib.check(rc, "naju_b200_fwd")
        if _check_status_enabled() and B * T * D > 0:
            st = lib.naju_b200_read_status(_ptr(scratch), _stream())
            _last_forms["fwd"] = lib.naju_b200_read_form(_ptr(scratch), _stream())
            if st != 0:
                raise RuntimeError(f"naju_b200_fwd device status {st} (bounded wait ran out)")
    if want_final and Np != N:
        hT = hT[..., :N].contiguous()
    return y, hT, pT, ckpt, d


def scan_backward(d, u, f_logit, i_logit, Bm, Cm, D_skip, h0, dy, dhT, ckpt, want_dh0=False):
    """Raw backward.  Returns (du, dfl, dil, dB, dC, dD, dh0|None).  `d` and `ckpt` are what
    scan_forward returned for the same tensors (NAJU_B200_FORM must not change in between: it
    decides whether fewer than 16 states are padded)."""
    lib = _lib.load()
    B, T, D = u.shape
    N = Bm.shape[-1]
    if _pad_to_group(u, Bm):
        Bm, Cm, h0, dhT = _pad_states(Bm), _pad_states(Cm), _pad_states(h0), _pad_states(dhT)
        d = _desc(u, f_logit, i_logit, Bm, Cm)
    Np = Bm.shape[-1]
    dev = u.device
    # (a time-contiguous u gets its gradient in the same layout: naju_b200.h, naju_scan_desc)
    du = torch.empty_strided((B, T, D), u.stride(), dtype=u.dtype, device=dev) if d.u_sd > 1 else \
        torch.empty((B, T, D), dtype=u.dtype, device=dev)
    dfl = torch.empty((B, T, D), dtype=f_logit.dtype, device=dev)
    dil = torch.empty((B, T, D), dtype=f_logit.dtype, device=dev)
    dB = torch.empty((B, T, Np), dtype=Bm.dtype, device=dev)
    dC = torch.empty((B, T, Np), dtype=Bm.dtype, device=dev)
    dD = torch.empty((D,), dtype=torch.float32, device=dev)
    dh0 = torch.empty((B, D, Np), dtype=torch.float32, device=dev) if want_dh0 else None
    scratch = _workspace(lib.naju_b200_bwd_scratch_bytes(d), dev)
    dy = dy.to(u.dtype).contiguous()
    with torch.cuda.device(dev):
        rc = lib.naju_b200_bwd(d, _ptr(u), _ptr(f_logit), _ptr(i_logit), _ptr(Bm), _ptr(Cm),
                               _ptr(D_skip), _ptr(h0), _ptr(dy), _ptr(dhT), _ptr(ckpt), _ptr(du),
                               _ptr(dfl), _ptr(dil), _ptr(dB), _ptr(dC), _ptr(dD), _ptr(dh0),
                               _ptr(scratch), _stream())
        _lib.check(rc, "naju_b200_bwd")
        if _check_status_enabled() and B * T * D > 0:
            st = lib.naju_b200_read_status(_ptr(scratch), _stream())
            _last_forms["bwd"] = lib.naju_b200_read_form(_ptr(scratch), _stream())
            if st != 0:
                raise RuntimeError(f"naju_b200_bwd device status {st} (bounded wait ran out)")
    if Np != N:
        dB, dC = dB[..., :N].contiguous(), dC[..., :N].contiguous()
        dh0 = None if dh0 is None else dh0[..., :N].contiguous()
    return du, dfl, dil, dB, dC, dD, dh0


class _NajuB200Scan(torch.autograd.Function):
    """Counterpart of _NajuCudaFn (naju/cuda/__init__.py:38-63) over the C ABI."""

    @staticmethod
    def forward(ctx, u, f_logit, i_logit, Bm, Cm, D_skip, h0, want_final):
        in_dtypes = (u.dtype, f_logit.dtype, i_logit.dtype, Bm.dtype, Cm.dtype, D_skip.dtype)
        pu, pf, pi, pB, pC, pD = _prepare(u, f_logit, i_logit, Bm, Cm, D_skip)
        B, T, D = pu.shape
        ph0 = _state_arg(h0, B, D, pB.shape[-1], "h0")
        y, hT, _, ckpt, d = scan_forward(pu, pf, pi, pB, pC, pD, ph0, want_final=want_final)
        ctx.save_for_backward(pu, pf, pi, pB, pC, pD, ph0, ckpt)
        ctx.desc = d
        ctx.in_dtypes = in_dtypes
        ctx.h0_dtype = None if h0 is None else h0.dtype
        ctx.want_final = want_final
        if want_final:
            return y, hT
        return y

    @staticmethod
    def backward(ctx, dy, dhT=None):
        pu, pf, pi, pB, pC, pD, ph0, ckpt = ctx.saved_tensors
        B, T, D = pu.shape
        N = pB.shape[-1]
        if dy is None:
            dy = torch.zeros_like(pu)
        pdhT = _state_arg(dhT, B, D, N, "dhT") if (ctx.want_final and dhT is not None) else None
        want_dh0 = ph0 is not None and ctx.needs_input_grad[6]
        du, dfl, dil, dB, dC, dD, dh0 = scan_backward(ctx.desc, pu, pf, pi, pB, pC, pD, ph0, dy,
                                                      pdhT, ckpt, want_dh0=want_dh0)
        t = ctx.in_dtypes
        return (du.to(t[0]), dfl.to(t[1]), dil.to(t[2]), dB.to(t[3]), dC.to(t[4]), dD.to(t[5]),
                None if dh0 is None else dh0.to(ctx.h0_dtype), None)


# ---------------------------------------------------------------------------------------------
# The same forward / backward as torch.library custom ops, so that torch.compile does not break
# the graph at the scan (the reference's scan is a graph break: naju/README.md:99-100) and
# NajuBlock(use_ckpt=True) (naju/mixer.py:139-141) composes.  Used while compiling; eager calls
# keep the autograd.Function above.
def _ckpt_bytes_formula(B, T, D, N):
    """Size of the checkpoint buffer (naju_b200_ckpt_bytes) as arithmetic that also works on the
    symbolic sizes of fake tensors."""
    NS = 16 if N <= 16 else 32 if N <= 32 else 64 if N <= 64 else 128
    TC = 64 if NS <= 32 else 32
    ntiles = ((T + TC - 1) // TC) * B * ((D + 127) // 128)
    a256 = lambda x: (x + 255) // 256 * 256
    return a256(ntiles * 128 * NS * 4) + a256(ntiles * 128 * 4) + 256


@torch.library.custom_op("naju_b200::scan_fwd", mutates_args=())
def _scan_fwd_op(u: torch.Tensor, f_logit: torch.Tensor, i_logit: torch.Tensor, Bm: torch.Tensor,
                 Cm: torch.Tensor, D_skip: torch.Tensor, h0: torch.Tensor,
                 want_final: bool) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    pu, pf, pi, pB, pC, pD = _prepare(u, f_logit, i_logit, Bm, Cm, D_skip)
    B, T, D = pu.shape
    ph0 = _state_arg(h0, B, D, pB.shape[-1], "h0") if h0.numel() else None
    y, hT, _, ckpt, _ = scan_forward(pu, pf, pi, pB, pC, pD, ph0, want_final=want_final)
    return y, (hT if want_final else y.new_empty(0, dtype=torch.float32)), ckpt


@_scan_fwd_op.register_fake
def _(u, f_logit, i_logit, Bm, Cm, D_skip, h0, want_final):
    B, T, D = u.shape
    N = Bm.shape[-1]
    hT = u.new_empty((B, D, N), dtype=torch.float32) if want_final else u.new_empty(0, dtype=torch.float32)
    # (fewer than 16 states may be padded to 16: the same rule as scan_forward, on the dtype
    # the prepared B and C take, see _prepare)
    bdt = Bm.dtype if (Bm.dtype == Cm.dtype and Bm.dtype in _DT) else torch.float32
    if _pad_to_group(u, u.new_empty((0, 0, N), dtype=bdt)):
        N = _GROUP
    ckpt = u.new_empty(_ckpt_bytes_formula(B, T, D, N), dtype=torch.uint8)
    return u.new_empty((B, T, D)), hT, ckpt


@torch.library.custom_op("naju_b200::scan_bwd", mutates_args=())
def _scan_bwd_op(u: torch.Tensor, f_logit: torch.Tensor, i_logit: torch.Tensor, Bm: torch.Tensor,
                 Cm: torch.Tensor, D_skip: torch.Tensor, h0: torch.Tensor, dy: torch.Tensor,
                 dhT: torch.Tensor, ckpt: torch.Tensor) -> list[torch.Tensor]:
    pu, pf, pi, pB, pC, pD = _prepare(u, f_logit, i_logit, Bm, Cm, D_skip)
    B, T, D = pu.shape
    N = pB.shape[-1]
    ph0 = _state_arg(h0, B, D, N, "h0") if h0.numel() else None
    pdhT = _state_arg(dhT, B, D, N, "dhT") if dhT.numel() else None
    d = _desc(pu, pf, pi, pB, pC)
    du, dfl, dil, dB, dC, dD, dh0 = scan_backward(d, pu, pf, pi, pB, pC, pD, ph0, dy, pdhT, ckpt,
                                                  want_dh0=ph0 is not None)
    if dh0 is None:
        dh0 = du.new_empty(0, dtype=torch.float32)
    # (the fake implementation promises contiguous gradients: a du that came back in the layout of a
    # time-contiguous u is made contiguous here)
    return [du.to(u.dtype).contiguous(), dfl.to(f_logit.dtype), dil.to(i_logit.dtype), dB.to(Bm.dtype), dC.to(Cm.dtype),
            dD.to(D_skip.dtype), dh0.to(h0.dtype)]


@_scan_bwd_op.register_fake
def _(u, f_logit, i_logit, Bm, Cm, D_skip, h0, dy, dhT, ckpt):
    return [torch.empty_like(u, memory_format=torch.contiguous_format),
            torch.empty_like(f_logit, memory_format=torch.contiguous_format),
            torch.empty_like(i_logit, memory_format=torch.contiguous_format),
            torch.empty_like(Bm, memory_format=torch.contiguous_format),
            torch.empty_like(Cm, memory_format=torch.contiguous_format),
            torch.empty_like(D_skip), torch.empty_like(h0)]


def _scan_op_setup(ctx, inputs, output):
    u, f_logit, i_logit, Bm, Cm, D_skip, h0, want_final = inputs
    ctx.save_for_backward(u, f_logit, i_logit, Bm, Cm, D_skip, h0, output[2])
    ctx.want_final = want_final


def _scan_op_backward(ctx, dy, dhT, _dckpt):
    u, f_logit, i_logit, Bm, Cm, D_skip, h0, ckpt = ctx.saved_tensors
    if dy is None:
        dy = torch.zeros_like(u)
    if dhT is None or not ctx.want_final:
        dhT = u.new_empty(0, dtype=torch.float32)
    du, dfl, dil, dB, dC, dD, dh0 = _scan_bwd_op(u, f_logit, i_logit, Bm, Cm, D_skip, h0, dy.contiguous(),
                                                 dhT, ckpt)
    return du, dfl, dil, dB, dC, dD, (dh0 if h0.numel() else None), None


_scan_fwd_op.register_autograd(_scan_op_backward, setup_context=_scan_op_setup)


def _scan_via_custom_op(u, f_logit, i_logit, B, C, D_skip, h0, want_final):
    h0t = h0 if h0 is not None else u.new_empty(0, dtype=torch.float32)
    y, hT, _ = _scan_fwd_op(u, f_logit, i_logit, B, C, D_skip, h0t, want_final)
    return (y, hT) if want_final else y


def naju_b200_scan(u, f_logit, i_logit, B, C, D_skip):
    """Backend callable with the reference's 6-tensor signature (naju/scan.py:3-5)."""
    return _NajuB200Scan.apply(u, f_logit, i_logit, B, C, D_skip, None, False)


def naju_scan(u, f_logit, i_logit, B, C, D_skip, backend=None, *, h0=None,
              return_final_state=False):
    """y = scan(u, f_logit, i_logit, B, C, D_skip) — drop-in for naju/scan.py:75-76.

    u, f_logit, i_logit [B,T,D]; B, C [B,T,N]; D_skip [D]; y [B,T,D] in u's dtype.
    Differentiable w.r.t. all six tensors (and h0).  With return_final_state=True returns
    (y, hT) where hT [B,D,N] fp32 is the state after the last step.
    """
    resolve_backend(backend)
    if torch.compiler.is_compiling():
        return _scan_via_custom_op(u, f_logit, i_logit, B, C, D_skip, h0, bool(return_final_state))
    return _NajuB200Scan.apply(u, f_logit, i_logit, B, C, D_skip, h0, bool(return_final_state))


@torch.no_grad()
def naju_scan_step(state, u_t, f_logit_t, i_logit_t, B_t, C_t, D_skip):
    """Single-token decode update: one iteration of naju/scan.py:87-91.

    state [B,D,N] fp32 (updated IN PLACE); u_t, f_logit_t, i_logit_t [B,D]; B_t, C_t [B,N].
    Returns (y_t [B,D] in u_t's dtype, state).
    """
    lib = _lib.load()
    if not state.is_cuda:
        raise RuntimeError("naju_b200 step needs CUDA tensors (there is no CPU fallback)")
    if state.dtype != torch.float32 or not state.is_contiguous():
        raise RuntimeError("state must be a contiguous fp32 [B, D, N] tensor")
    Bsz, D, N = state.shape
    pu, pf, pi, pB, pC, pD = _prepare(u_t.unsqueeze(1), f_logit_t.unsqueeze(1),
                                      i_logit_t.unsqueeze(1), B_t.unsqueeze(1), C_t.unsqueeze(1),
                                      D_skip)
    d = _desc(pu, pf, pi, pB, pC)
    d.T = 1
    d.u_sb, d.fl_sb, d.il_sb = max(d.u_sb, D), max(d.fl_sb, D), max(d.il_sb, D)
    d.bm_sb, d.cm_sb = max(d.bm_sb, N), max(d.cm_sb, N)
    y = torch.empty((Bsz, D), dtype=pu.dtype, device=state.device)
    with torch.cuda.device(state.device):
        rc = lib.naju_b200_step(d, _ptr(state), _ptr(pu), _ptr(pf), _ptr(pi), _ptr(pB), _ptr(pC),
                                _ptr(pD), _ptr(y), _stream())
    _lib.check(rc, "naju_b200_step")
    return y, state
