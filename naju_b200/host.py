"""Scan over HOST-resident tensors: batch rows streamed through the GPU.

The scan has no dependency between batch rows, so when the six inputs (and dy) live in pinned host
memory the copies can overlap the kernels and each other: while rows j are in the forward/backward
kernels, rows j+1 are on their way in and the results of rows j-1 on their way out (PCIe is full
duplex).  Three CUDA streams (in, compute, out) and a small ring of device buffers do this; every
kernel call goes through the same C ABI as `naju_scan`.  The reference has no counterpart (its
mixer keeps everything on the device, naju/mixer.py:111-124); this is for callers whose
activations are off-loaded, and it is what `bench.py` times as the end-to-end figure.
"""
import torch

from .scan import _prepare, scan_backward, scan_forward

_SLOTS = 3
_streams = {}


def _get_streams(dev):
    key = (dev.type, dev.index)
    if key not in _streams:
        _streams[key] = tuple(torch.cuda.Stream(device=dev) for _ in range(3))
    return _streams[key]


def _pinned_like(shape, dtype):
    return torch.empty(shape, dtype=dtype).pin_memory()


def scan_fwd_bwd_host(u, f_logit, i_logit, B, C, D_skip, dy, *, rows_per_chunk=1, time_splits=1, device=None,
                      out=None):
    """Forward and backward of the scan for host tensors.

    u, f_logit, i_logit, dy: [B, T, D]; B, C: [B, T, N] (pinned host memory for the copies to be
    asynchronous); D_skip: [D], host or device.  Returns a dict of host tensors
    {y, du, dfl, dil, dB, dC, dD}: y and du in u's dtype, the logit gradients in the logits' dtype,
    dB/dC in B's dtype, dD fp32.  `out` may hand in such a dict (pinned) to be filled again.
    With time_splits = K > 1 (and rows_per_chunk = 1) every row is further cut into K contiguous
    time segments: the forward runs segment by segment with the final state of one as the initial
    state of the next, the backward runs them in reverse with the adjoint of the initial state
    handed back the same way (the composition law of naju/tests/test_affine_chunk.py:47-78), and
    copies move at segment granularity, which shortens the unoverlapped head and tail of the
    pipeline.  The call returns when all copies have been enqueued; the current stream then waits
    for them, so a synchronize of the current stream (or device) makes the host tensors valid.
    Same semantics as naju_scan (naju/scan.py:75-93) + autograd; zero initial state.
    """
    if not torch.cuda.is_available():
        raise RuntimeError("naju_b200 host pipeline needs a CUDA device (there is no CPU fallback)")
    for t in (u, f_logit, i_logit, B, C, dy):
        if t.is_cuda:
            raise ValueError("scan_fwd_bwd_host takes host tensors (use naju_scan for device tensors)")
    if u.dim() != 3 or f_logit.shape != u.shape or i_logit.shape != u.shape or dy.shape != u.shape:
        raise ValueError("u, f_logit, i_logit, dy must all be [B, T, D]")
    if B.dim() != 3 or B.shape != C.shape or B.shape[:2] != u.shape[:2]:
        raise ValueError("B and C must both be [B, T, N] matching u's batch and time")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    nb, T, D = u.shape
    N = B.shape[-1]
    rows = max(1, min(int(rows_per_chunk), nb))
    nchunk = (nb + rows - 1) // rows
    s_in, s_cmp, s_out = _get_streams(dev)
    cur = torch.cuda.current_stream(dev)

    ins = (u, f_logit, i_logit, B, C, dy)
    if out is None:
        out = {"y": _pinned_like(u.shape, u.dtype), "du": _pinned_like(u.shape, u.dtype),
               "dfl": _pinned_like(u.shape, f_logit.dtype), "dil": _pinned_like(u.shape, i_logit.dtype),
               "dB": _pinned_like(B.shape, B.dtype), "dC": _pinned_like(C.shape, C.dtype),
               "dD": _pinned_like((D,), torch.float32)}
    with torch.cuda.device(dev):
        for s in (s_in, s_cmp, s_out):
            s.wait_stream(cur)
        with torch.cuda.stream(s_cmp):
            Dk = D_skip.detach().to(dev, torch.float32)
            dD_acc = torch.zeros(D, dtype=torch.float32, device=dev)
        slots = []
        with torch.cuda.stream(s_in):
            for _ in range(min(_SLOTS, nchunk)):
                slots.append([torch.empty((rows,) + tuple(t.shape[1:]), dtype=t.dtype, device=dev) for t in ins])
        ev_in = [torch.cuda.Event() for _ in range(nchunk)]
        ev_cmp = [torch.cuda.Event() for _ in range(nchunk)]
        K = max(1, int(time_splits)) if rows == 1 else 1
        K = min(K, max(1, T // 256))  # segments shorter than a few chunks only add launches
        seg = [(k * T // K, (k + 1) * T // K) for k in range(K)]
        names = ("y", "du", "dfl", "dil", "dB", "dC")

        def to_host(name, t, r0, r1, t0, t1):
            dst = out[name][r0:r1, t0:t1]
            dst.copy_(t.to(dst.dtype) if t.dtype != dst.dtype else t, non_blocking=True)
            t.record_stream(s_out)

        for j in range(nchunk):
            r0, r1 = j * rows, min((j + 1) * rows, nb)
            n = r1 - r0
            slot = slots[j % len(slots)]
            ev_seg = [torch.cuda.Event() for _ in range(K)]
            with torch.cuda.stream(s_in):
                if j >= len(slots):
                    s_in.wait_event(ev_cmp[j - len(slots)])  # the kernels have read this slot's inputs
                for k, (t0, t1) in enumerate(seg):
                    for dst, src in zip(slot, ins):
                        dst[:n, t0:t1].copy_(src[r0:r1, t0:t1], non_blocking=True)
                    ev_seg[k].record(s_in)
                ev_in[j].record(s_in)
            fwd = []
            ev_f = [torch.cuda.Event() for _ in range(K)]
            ev_b = [torch.cuda.Event() for _ in range(K)]
            grads = [None] * K
            with torch.cuda.stream(s_cmp):
                h_prev = None
                for k, (t0, t1) in enumerate(seg):
                    s_cmp.wait_event(ev_seg[k])
                    du_, fl_, il_, b_, c_, dy_ = (t[:n, t0:t1] for t in slot)
                    pu, pf, pi, pb, pc, pD = _prepare(du_, fl_, il_, b_, c_, Dk)
                    y, hT, _, ckpt, desc = scan_forward(pu, pf, pi, pb, pc, pD, h0=h_prev, want_final=K > 1)
                    fwd.append((pu, pf, pi, pb, pc, pD, h_prev, dy_, ckpt, desc, y))
                    h_prev = hT
                    ev_f[k].record(s_cmp)
                lam = None
                for k in range(K - 1, -1, -1):
                    pu, pf, pi, pb, pc, pD, h0k, dy_, ckpt, desc, _ = fwd[k]
                    g = scan_backward(desc, pu, pf, pi, pb, pc, pD, h0k, dy_, lam, ckpt, want_dh0=k > 0)
                    lam = g[6]
                    dD_acc += g[5]
                    grads[k] = g
                    ev_b[k].record(s_cmp)
                ev_cmp[j].record(s_cmp)
            with torch.cuda.stream(s_out):
                for k, (t0, t1) in enumerate(seg):
                    s_out.wait_event(ev_f[k])
                    to_host("y", fwd[k][10], r0, r1, t0, t1)
                for k in range(K - 1, -1, -1):
                    t0, t1 = seg[k]
                    s_out.wait_event(ev_b[k])
                    for name, t in zip(names[1:], grads[k][:5]):
                        to_host(name, t, r0, r1, t0, t1)
        with torch.cuda.stream(s_out):
            s_out.wait_stream(s_cmp)
            out["dD"].copy_(dD_acc, non_blocking=True)
            dD_acc.record_stream(s_out)
        for slot in slots:
            for t in slot:
                t.record_stream(s_cmp)
        cur.wait_stream(s_out)
        cur.wait_stream(s_cmp)
        cur.wait_stream(s_in)
    return out
