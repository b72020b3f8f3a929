"""Multi-GPU forms of the scan (one process per GPU, torch.distributed for the plumbing).

Batch sharding needs nothing from this module but `shard_batch`: every (batch row, channel) pair
is an independent recurrence, so each rank simply calls `naju_scan` on its rows; there is no
collective on the data path.

Channel sharding, for batches smaller than the number of GPUs (`naju_scan_channel_sharded`):
rank r holds the channel slice [r*D/R, (r+1)*D/R) of u, the two logit tensors, D_skip and y,
and a full copy of B and C.  The forward needs no exchange.  In the backward every gradient
but two is local to the slice; dB and dC sum over channels, so each rank's are partial sums
over its own channels and one fp32 all-reduce of the two [B,T,N] tensors completes them
(2 * B*T*N*4 bytes: 16.8 MB at B=8, T=16384, N=16).

Time sharding, for sequences too long for one GPU: rank r holds the time slice
[r*T/R, (r+1)*T/R) of every tensor.  The recurrence is affine in the state, so a slice is
summarised by (S_r, P_r) = (its final state from a zero start, the product of its retention
gates), and only those two small tensors cross NVLink:

  1. every rank scans its slice from a zero state (rank 0: from h0), in parallel;
  2. every rank learns every slice's (S_r, P_r) with ONE all_gather ([B,D,N] + [B,D] fp32 per
     rank, received into this rank's own memory) and folds the slices before its own,
     h_in,r+1 = P_r * h_in,r + S_r, locally -- no serial chain of hops, no host round trip
     (`handoff="chain"` keeps the older send/recv chain with a shape header per hop);
  3. ranks whose carry-in is non-zero scan again from the true h_in -- under no_grad only the
     leading part of the slice, up to the chunk where the cumulative retention product has
     decayed below 1e-30 in every channel and the carry can no longer change y.
The backward mirrors this in reverse time with the adjoint carry and yields dh0 on rank 0.

The reference has no multi-GPU code at all; the single-slice semantics are those of
naju/scan.py:79-93 and the composition law is the one naju/tests/test_affine_chunk.py:47-78
checks (scan [0,s) then [s,T) from the first part's final state == scan [0,T)).
"""
import torch
import torch.distributed as dist

_DECAY_DEAD = 1e-30


class CudaLocalScan:
    """Local slice scan on this rank's GPU through the C ABI."""

    def forward(self, u, fl, il, Bm, Cm, Dk, h0, need_ckpt=True):
        from . import scan as S
        pu, pf, pi, pB, pC, pD = S._prepare(u, fl, il, Bm, Cm, Dk)
        ph0 = S._state_arg(h0, pu.shape[0], pu.shape[2], pB.shape[-1], "h0")
        y, hT, pT, ckpt, d = S.scan_forward(pu, pf, pi, pB, pC, pD, ph0, want_final=True,
                                            want_decay=True)
        return y, hT, pT, (pu, pf, pi, pB, pC, pD, ph0, ckpt, d)

    def backward(self, ctx, dy, dhT):
        from . import scan as S
        pu, pf, pi, pB, pC, pD, ph0, ckpt, d = ctx
        # (the terminal adjoint may arrive as a strided view, e.g. a channel slice)
        pdhT = S._state_arg(dhT, pu.shape[0], pu.shape[2], pB.shape[-1], "dhT")
        return S.scan_backward(d, pu, pf, pi, pB, pC, pD, ph0, dy, pdhT, ckpt, want_dh0=True)

    def dead_prefix_len(self, ctx, T):
        """Number of leading steps after which the carry-in cannot influence y any more
        (a multiple of the chunk length; T if the retention never dies out)."""
        from . import _lib
        pu, _, _, pB, _, _, _, ckpt, d = ctx
        lib = _lib.load()
        tc = lib.naju_b200_chunk_len(d)
        off = lib.naju_b200_ckpt_decay_offset(d)
        nchunks = (T + tc - 1) // tc
        per_chunk = pu.shape[0] * ((pu.shape[2] + 127) // 128) * 128
        P = ckpt[off:off + nchunks * per_chunk * 4].view(torch.float32).view(nchunks, per_chunk)
        # padded channels carry sigmoid(0)^t, which dies out quickly too, so the max is safe
        alive = (P.amax(dim=1) >= _DECAY_DEAD).to(torch.int32)
        n_alive = int(alive.sum().item())  # P is non-increasing in the chunk index
        return min(T, (n_alive + 1) * tc)


def _group_info(group):
    return dist.get_rank(group), dist.get_world_size(group)


def _peer(group, r):
    return dist.get_global_rank(group, r) if group is not None else r


def _check_header(mine, theirs, what):
    if not torch.equal(mine.cpu(), theirs.cpu()):
        raise RuntimeError(f"time-sharded scan: {what} hand-off shape mismatch "
                           f"(expected {mine.tolist()}, peer sent {theirs.tolist()})")


def _send_state(t, dst, group):
    hdr = torch.tensor(list(t.shape), dtype=torch.int64, device=t.device)
    dist.send(hdr, _peer(group, dst), group=group)
    dist.send(t.contiguous(), _peer(group, dst), group=group)


def _recv_state(like, src, group):
    hdr = torch.empty(like.dim(), dtype=torch.int64, device=like.device)
    dist.recv(hdr, _peer(group, src), group=group)
    _check_header(torch.tensor(list(like.shape), dtype=torch.int64), hdr, "state")
    out = torch.empty_like(like)
    dist.recv(out, _peer(group, src), group=group)
    return out


def chain_forward(S, P, h0, group):
    """Step 2: returns (h_in, h_out) of this rank.  S [B,D,N] is the slice's final state from a
    zero start (on rank 0: from h0, which it therefore already contains), P [B,D] fp32."""
    rank, world = _group_info(group)
    if rank == 0:
        h_in = torch.zeros_like(S) if h0 is None else h0.to(S.dtype)
        h_out = S
    else:
        h_in = _recv_state(S, rank - 1, group)
        h_out = P.unsqueeze(-1) * h_in + S
    if rank < world - 1:
        _send_state(h_out, rank + 1, group)
    return h_in, h_out


def gather_forward(S, P, h0, group):
    """Step 2 with one collective: all ranks' (S, P) are gathered and the carry entering this
    rank's slice is the fold of the slices before it.  Returns (h_in, h_out) like chain_forward."""
    rank, world = _group_info(group)
    pack = torch.cat([S.reshape(S.shape[0], -1), P.reshape(P.shape[0], -1)], dim=1).contiguous()
    got = [torch.empty_like(pack) for _ in range(world)]
    dist.all_gather(got, pack, group=group)
    nS = S[0].numel()
    h = torch.zeros_like(S) if h0 is None else h0.to(S.dtype)   # (S of rank 0 already contains h0)
    h_in = h
    for k in range(rank):
        Sk = got[k][:, :nS].reshape(S.shape)
        Pk = got[k][:, nS:].reshape(P.shape)
        h_in = Sk if k == 0 else Pk.unsqueeze(-1) * h_in + Sk
    if rank == 0:
        return h, S
    return h_in, P.unsqueeze(-1) * h_in + S


def gather_backward(L, P, group):
    """Adjoint hand-off with one collective; returns (lam_in, lam_out) like chain_backward."""
    rank, world = _group_info(group)
    pack = torch.cat([L.reshape(L.shape[0], -1), P.reshape(P.shape[0], -1)], dim=1).contiguous()
    got = [torch.empty_like(pack) for _ in range(world)]
    dist.all_gather(got, pack, group=group)
    nL = L[0].numel()
    lam_in = torch.zeros_like(L)
    for k in range(world - 1, rank, -1):
        Lk = got[k][:, :nL].reshape(L.shape)
        Pk = got[k][:, nL:].reshape(P.shape)
        lam_in = Pk.unsqueeze(-1) * lam_in + Lk
    return lam_in, P.unsqueeze(-1) * lam_in + L


def chain_backward(L, P, group):
    """Adjoint chain.  L [B,D,N] = this slice's dh0 for a zero adjoint from later slices.
    Returns (lam_in, lam_out): the adjoint entering this slice from the future (zero on the
    last rank) and the one handed to the previous rank (on rank 0: the gradient of h0)."""
    rank, world = _group_info(group)
    if rank == world - 1:
        lam_in = torch.zeros_like(L)
    else:
        lam_in = _recv_state(L, rank + 1, group)
    lam_out = P.unsqueeze(-1) * lam_in + L
    if rank > 0:
        _send_state(lam_out, rank - 1, group)
    return lam_in, lam_out


class _TimeShardedScan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, u, fl, il, Bm, Cm, Dk, h0, group, local, want_final, handoff):
        rank, world = _group_info(group)
        T = u.shape[1]
        needs_grad = any(ctx.needs_input_grad[:7])
        first_h0 = h0 if rank == 0 else None
        y, S, P, lctx = local.forward(u, fl, il, Bm, Cm, Dk, first_h0)
        h_in, h_out = (gather_forward if handoff == "all_gather" else chain_forward)(S, P, first_h0, group)
        if rank > 0:   # (no look at the carry's values: that would be a host round trip)
            if needs_grad:
                y, _, _, lctx = local.forward(u, fl, il, Bm, Cm, Dk, h_in)
            else:
                n = local.dead_prefix_len(lctx, T) if hasattr(local, "dead_prefix_len") else T
                y_fix, _, _, _ = local.forward(u[:, :n], fl[:, :n], il[:, :n], Bm[:, :n], Cm[:, :n],
                                               Dk, h_in)
                y = y.clone() if not y.is_contiguous() else y
                y[:, :n] = y_fix
        ctx.local, ctx.lctx, ctx.group, ctx.P = local, lctx, group, P
        ctx.want_final, ctx.handoff = want_final, handoff
        ctx.has_h0 = h0 is not None
        ctx.in_dtypes = tuple(t.dtype for t in (u, fl, il, Bm, Cm, Dk))
        ctx.mark_non_differentiable(P)
        if want_final:
            return y, h_out, P
        return y

    @staticmethod
    def backward(ctx, dy, dh_out=None, _dP=None):
        local, group, P = ctx.local, ctx.group, ctx.P
        rank, world = _group_info(group)
        dy = dy.contiguous()
        term = dh_out if (ctx.want_final and dh_out is not None) else None
        # pass A: zero adjoint from the future (plus this rank's own terminal adjoint)
        gA = local.backward(ctx.lctx, dy, term)
        lam_in, lam_out = (gather_backward if ctx.handoff == "all_gather" else chain_backward)(gA[6], P, group)
        g = gA
        if rank < world - 1:
            total = lam_in if term is None else lam_in + term.to(lam_in.dtype)
            g = local.backward(ctx.lctx, dy, total)
            lam_out = g[6]
        t = ctx.in_dtypes
        dh0 = lam_out if (ctx.has_h0 and rank == 0) else None
        return (g[0].to(t[0]), g[1].to(t[1]), g[2].to(t[2]), g[3].to(t[3]), g[4].to(t[4]),
                g[5].to(t[5]), dh0, None, None, None, None)


def naju_scan_time_sharded(u, f_logit, i_logit, B, C, D_skip, group=None, *, h0=None,
                           return_final_state=False, local=None, handoff="all_gather"):
    """Scan of a sequence whose time axis is split across the ranks of `group`.

    Every rank passes ITS slice ([B, T_r, D] / [B, T_r, N]) and gets its slice of y.  `h0`
    (rank 0 only) is the global initial state.  With return_final_state=True also returns
    (state at the end of this rank's slice, product of the retention gates over the slice);
    the global final state is the one on the last rank.  Gradients: each rank receives the
    gradients of its own slices; D_skip's gradient is this rank's partial sum (sum over ranks
    for the total, like any replicated parameter); dh0 arrives on rank 0.  `handoff` selects how
    the slice summaries travel: "all_gather" (one collective, default) or "chain" (send/recv
    from rank to rank with a shape header per hop).
    """
    if not dist.is_initialized():
        raise RuntimeError("naju_scan_time_sharded needs an initialised torch.distributed group")
    if handoff not in ("all_gather", "chain"):
        raise ValueError("handoff must be 'all_gather' or 'chain'")
    local = local or CudaLocalScan()
    return _TimeShardedScan.apply(u, f_logit, i_logit, B, C, D_skip, h0, group, local,
                                  bool(return_final_state), handoff)


class _ChannelShardedScan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, u, fl, il, Bm, Cm, Dk, h0, group, local, want_final, reduce_bc):
        y, hT, _, lctx = local.forward(u, fl, il, Bm, Cm, Dk, h0)
        ctx.local, ctx.lctx, ctx.group = local, lctx, group
        ctx.want_final, ctx.reduce_bc, ctx.has_h0 = want_final, reduce_bc, h0 is not None
        ctx.in_dtypes = tuple(t.dtype for t in (u, fl, il, Bm, Cm, Dk))
        if want_final:
            return y, hT
        return y

    @staticmethod
    def backward(ctx, dy, dhT=None):
        term = dhT if (ctx.want_final and dhT is not None) else None
        du, dfl, dil, dB, dC, dD, dh0 = ctx.local.backward(ctx.lctx, dy.contiguous(), term)
        if ctx.reduce_bc:
            # partial sums over this rank's channels -> sums over all channels, in fp32, one
            # collective for both tensors
            both = torch.stack([dB.to(torch.float32), dC.to(torch.float32)])
            dist.all_reduce(both, op=dist.ReduceOp.SUM, group=ctx.group)
            dB, dC = both[0], both[1]
        t = ctx.in_dtypes
        return (du.to(t[0]), dfl.to(t[1]), dil.to(t[2]), dB.to(t[3]), dC.to(t[4]), dD.to(t[5]),
                dh0 if ctx.has_h0 else None, None, None, None, None)


def naju_scan_channel_sharded(u, f_logit, i_logit, B, C, D_skip, group=None, *, h0=None,
                              return_final_state=False, reduce_bc=True, local=None):
    """Scan whose CHANNEL axis is split across the ranks of `group` (for batches smaller than
    the group).

    Every rank passes its channel slice of u, f_logit, i_logit ([B, T, D_r]), D_skip ([D_r]) and
    h0 ([B, D_r, N]), and the full B and C ([B, T, N], the same on every rank); it gets its slice
    of y (and of the final state).  The forward exchanges nothing.  Gradients of the sliced
    tensors are local.  dB and dC sum over channels: with reduce_bc=True (default) they are
    completed by one fp32 all-reduce over the group, so every rank returns the full gradient of
    its copy of B and C; with reduce_bc=False each rank returns its partial sums and the caller
    adds them (e.g. together with other gradients of a replicated tensor).
    """
    if reduce_bc and not dist.is_initialized():
        raise RuntimeError("naju_scan_channel_sharded(reduce_bc=True) needs an initialised torch.distributed group")
    local = local or CudaLocalScan()
    return _ChannelShardedScan.apply(u, f_logit, i_logit, B, C, D_skip, h0, group, local,
                                     bool(return_final_state), bool(reduce_bc))


def shard_channels(t, rank, world, dim=-1, multiple=128):
    """Channels of `t` along `dim` owned by `rank`: contiguous slices whose length is a multiple of
    `multiple` (the kernels tile channels by 128) except possibly the last."""
    D = t.shape[dim]
    per = (D + world - 1) // world
    per = (per + multiple - 1) // multiple * multiple
    lo, hi = min(D, rank * per), min(D, (rank + 1) * per)
    return t.narrow(dim, lo, hi - lo)


def shard_batch(t, rank, world):
    """Rows of a [B, ...] tensor owned by `rank` under batch sharding (no collective needed)."""
    B = t.shape[0]
    per = (B + world - 1) // world
    return t[rank * per:min(B, (rank + 1) * per)]
