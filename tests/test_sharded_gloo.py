"""Host logic of the multi-GPU forms, run as gloo ranks on CPU (world size 2 and 3).

The per-rank slice scan is injected: here it is the CPU oracle (test infrastructure), on a GPU
box it is the CUDA path.  What is under test is the hand-off: the forward carry chain, the
adjoint chain, the shape header, and that a rank which dies or never sends makes its peer fail
with an error inside the process-group timeout instead of hanging.
"""
import datetime
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


class OracleLocalScan:
    """Slice scan backed by the CPU oracle (fp64 arithmetic), same interface as CudaLocalScan."""

    def forward(self, u, fl, il, Bm, Cm, Dk, h0, need_ckpt=True):
        import oracle
        a = [t.detach().numpy() for t in (u, fl, il, Bm, Cm, Dk)]
        h0n = None if h0 is None else h0.detach().numpy()
        y, hT = oracle.oracle_fwd(*a, h0=h0n, return_final_state=True)
        P = np.prod(1.0 / (1.0 + np.exp(-a[1].astype(np.float64))), axis=1).astype(np.float32)
        return torch.tensor(y), torch.tensor(hT), torch.tensor(P), (a, h0n)

    def backward(self, ctx, dy, dhT):
        import oracle
        a, h0n = ctx
        g = oracle.oracle_bwd(*a, dy.numpy(), h0=h0n, dhT=None if dhT is None else dhT.numpy())
        return tuple(torch.tensor(g[k]) for k in ("du", "dfl", "dil", "dB", "dC", "dD", "dh0"))


def _init(rank, world, port, timeout_s=60):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=timeout_s))


def _worker_parity(rank, world, port, q, handoff="all_gather"):
    import oracle
    from naju_b200.sharded import naju_scan_time_sharded
    _init(rank, world, port)
    B, T, D, N = 2, 30 * world, 12, 16
    d = oracle.make_inputs(B, T, D, N, seed=4, f_shift=3.0, d_skip_scale=0.01, with_h0=True)
    lo, hi = rank * T // world, (rank + 1) * T // world
    t = {k: torch.tensor(d[k][:, lo:hi]).requires_grad_(True) for k in ("u", "fl", "il", "Bm", "Cm")}
    Dk = torch.tensor(d["Dskip"]).requires_grad_(True)
    h0 = torch.tensor(d["h0"]).requires_grad_(True) if rank == 0 else None
    y, h_end, _ = naju_scan_time_sharded(t["u"], t["fl"], t["il"], t["Bm"], t["Cm"], Dk, None, h0=h0,
                                         return_final_state=True, local=OracleLocalScan(), handoff=handoff)
    outs = [y]
    grads = [torch.tensor(d["dy"][:, lo:hi])]
    if rank == world - 1:
        outs.append(h_end)
        grads.append(torch.tensor(d["dhT"]))
    torch.autograd.backward(outs, grads)
    res = dict(rank=rank, y=y.detach().numpy(), h_end=h_end.detach().numpy(),
               dD=Dk.grad.numpy(), **{"d" + k: t[k].grad.numpy() for k in t})
    if rank == 0:
        res["dh0"] = h0.grad.numpy()
    q.put(res)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,handoff", [(2, "all_gather"), (3, "all_gather"), (3, "chain")])
def test_time_sharded_matches_unsharded_oracle(world, handoff):
    import oracle
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_parity, args=(r, world, port, q, handoff)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=120) for _ in range(world)], key=lambda r: r["rank"])
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    B, T, D, N = 2, 30 * world, 12, 16
    d = oracle.make_inputs(B, T, D, N, seed=4, f_shift=3.0, d_skip_scale=0.01, with_h0=True)
    a = (d["u"], d["fl"], d["il"], d["Bm"], d["Cm"], d["Dskip"])
    y, hT = oracle.oracle_fwd(*a, h0=d["h0"], return_final_state=True)
    g = oracle.oracle_bwd(*a, d["dy"], h0=d["h0"], dhT=d["dhT"])
    cat = lambda k: np.concatenate([r[k] for r in res], axis=1)
    assert oracle.rel_l2(cat("y"), y) < 1e-6
    assert oracle.rel_l2(res[-1]["h_end"], hT) < 1e-6
    for k, gk in (("du", "du"), ("dfl", "dfl"), ("dil", "dil"), ("dBm", "dB"), ("dCm", "dC")):
        assert oracle.rel_l2(cat(k), g[gk]) < 2e-6, k
    assert oracle.rel_l2(sum(r["dD"] for r in res), g["dD"]) < 2e-6
    assert oracle.rel_l2(res[0]["dh0"], g["dh0"]) < 2e-6


def _worker_channels(rank, world, port, q, reduce_bc):
    import oracle
    from naju_b200.sharded import naju_scan_channel_sharded, shard_channels
    _init(rank, world, port)
    B, T, D, N = 2, 40, 20, 16
    d = oracle.make_inputs(B, T, D, N, seed=6, f_shift=2.0, d_skip_scale=0.01, with_h0=True)
    sl = lambda a, dim: shard_channels(torch.tensor(a), rank, world, dim=dim, multiple=4).clone()
    t = {k: sl(d[k], 2).requires_grad_(True) for k in ("u", "fl", "il")}
    t["Bm"], t["Cm"] = (torch.tensor(d[k]).requires_grad_(True) for k in ("Bm", "Cm"))
    Dk = sl(d["Dskip"], 0).requires_grad_(True)
    h0 = sl(d["h0"], 1).requires_grad_(True)
    y, hT = naju_scan_channel_sharded(t["u"], t["fl"], t["il"], t["Bm"], t["Cm"], Dk, None, h0=h0,
                                      return_final_state=True, reduce_bc=reduce_bc, local=OracleLocalScan())
    torch.autograd.backward([y, hT], [sl(d["dy"], 2), sl(d["dhT"], 1)])
    q.put(dict(rank=rank, y=y.detach().numpy(), hT=hT.detach().numpy(), dD=Dk.grad.numpy(),
               dh0=h0.grad.numpy(), **{"d" + k: t[k].grad.numpy() for k in t}))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,reduce_bc", [(2, True), (3, True), (2, False)])
def test_channel_sharded_matches_unsharded_oracle(world, reduce_bc):
    """Channel slices per rank, B and C replicated: y, the states and the sliced gradients are
    local; dB / dC are partial sums over the rank's channels, completed by one all-reduce
    (reduce_bc=True: every rank holds the full sums) or left to the caller (False: they add up)."""
    import oracle
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_channels, args=(r, world, port, q, reduce_bc)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=120) for _ in range(world)], key=lambda r: r["rank"])
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    B, T, D, N = 2, 40, 20, 16
    d = oracle.make_inputs(B, T, D, N, seed=6, f_shift=2.0, d_skip_scale=0.01, with_h0=True)
    a = (d["u"], d["fl"], d["il"], d["Bm"], d["Cm"], d["Dskip"])
    y, hT = oracle.oracle_fwd(*a, h0=d["h0"], return_final_state=True)
    g = oracle.oracle_bwd(*a, d["dy"], h0=d["h0"], dhT=d["dhT"])
    cat = lambda k, ax: np.concatenate([r[k] for r in res], axis=ax)
    assert oracle.rel_l2(cat("y", 2), y) < 1e-6
    assert oracle.rel_l2(cat("hT", 1), hT) < 1e-6
    for k, gk in (("du", "du"), ("dfl", "dfl"), ("dil", "dil")):
        assert oracle.rel_l2(cat(k, 2), g[gk]) < 2e-6, k
    assert oracle.rel_l2(cat("dD", 0), g["dD"]) < 2e-6
    assert oracle.rel_l2(cat("dh0", 1), g["dh0"]) < 2e-6
    for k, gk in (("dBm", "dB"), ("dCm", "dC")):
        if reduce_bc:
            for r in res:
                assert oracle.rel_l2(r[k], g[gk]) < 2e-6, k
        else:
            assert oracle.rel_l2(sum(r[k] for r in res), g[gk]) < 2e-6, k


def _worker_fault(rank, world, port, q, mode):
    from naju_b200.sharded import chain_forward
    try:
        _init(rank, world, port, timeout_s=120)          # generous: process start-up is slow
        grp = dist.new_group(ranks=list(range(world)), timeout=datetime.timedelta(seconds=5))
        dist.barrier()
        S = torch.ones(2, 4, 16)
        P = torch.full((2, 4), 0.5)
        if mode == "wrong_shape" and rank == 0:
            chain_forward(torch.ones(2, 5, 16), torch.full((2, 5), 0.5), None, grp)
            q.put((rank, "sent"))
        elif mode == "peer_exits" and rank == 0:
            q.put((rank, "exited"))   # leaves between steps, nothing in flight
            q.close()
            q.join_thread()
            os._exit(0)
        else:
            chain_forward(S, P, None, grp)
            q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, "error: " + type(e).__name__ + ": " + str(e)[:80]))
    q.close()
    q.join_thread()                              # flush before the hard exit below
    os._exit(0)


@pytest.mark.parametrize("mode", ["wrong_shape", "peer_exits"])
def test_hand_off_failures_surface_as_errors_not_hangs(mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_fault, args=(r, 2, port, q, mode)) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    try:
        while 1 not in got:                      # only the receiving rank's verdict matters
            r, msg = q.get(timeout=90)
            got[r] = msg
    finally:
        for p in procs:                          # the sender may sit in a blocked send: end it
            p.join(1)
            if p.is_alive():
                p.terminate()
                p.join(10)
    assert got[1].startswith("error"), got     # the receiving rank raised instead of hanging
    if mode == "wrong_shape":
        assert "mismatch" in got[1]


def test_shard_channels_partitions_in_tile_multiples():
    from naju_b200.sharded import shard_channels
    t = torch.arange(2 * 3 * 1000).view(2, 3, 1000)
    parts = [shard_channels(t, r, 3) for r in range(3)]
    assert torch.equal(torch.cat(parts, dim=-1), t)
    assert [p.shape[-1] for p in parts] == [384, 384, 232]
    parts = [shard_channels(t, r, 8, dim=2, multiple=128) for r in range(8)]
    assert torch.equal(torch.cat(parts, dim=2), t)
    assert [p.shape[2] for p in parts] == [128] * 7 + [104]


def test_shard_batch_partitions_rows():
    from naju_b200.sharded import shard_batch
    t = torch.arange(10).view(10, 1)
    parts = [shard_batch(t, r, 4) for r in range(4)]
    assert torch.equal(torch.cat(parts), t)
    assert [p.shape[0] for p in parts] == [3, 3, 3, 1]
