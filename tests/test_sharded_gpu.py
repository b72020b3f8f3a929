"""Time-sharded scan with the CUDA slice scan: single-rank group on one GPU, and (where the
box has two GPUs) a real two-rank NCCL hand-off checked against the unsharded oracle."""
import datetime
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def test_single_rank_group_equals_plain_scan_and_dead_prefix():
    from naju_b200 import naju_scan
    from naju_b200.sharded import CudaLocalScan, naju_scan_time_sharded
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(_free_port())
    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        B, T, D, N = 2, 700, 192, 16
        d = oracle.make_inputs(B, T, D, N, seed=8, f_shift=-1.0)   # f ~ 0.27: dies within ~60 steps
        t = [torch.tensor(d[k], device="cuda") for k in ("u", "fl", "il", "Bm", "Cm", "Dskip")]
        with torch.no_grad():
            y1 = naju_scan_time_sharded(*t)
            y0 = naju_scan(*t)
        assert oracle.rel_l2(y1.cpu().numpy(), y0.cpu().numpy()) < 2e-6
        loc = CudaLocalScan()
        _, _, pT, ctx = loc.forward(*t, None)
        n = loc.dead_prefix_len(ctx, T)
        f = 1.0 / (1.0 + np.exp(-d["fl"].astype(np.float64)))
        cum = np.cumprod(f, axis=1).max(axis=(0, 2))           # [T] max over batch and channels
        first_dead = int(np.argmax(cum < 1e-30)) if (cum < 1e-30).any() else T
        assert first_dead <= n <= min(T, first_dead + 2 * 64 + 64)   # chunk granularity (64 steps)
        assert n < T
    finally:
        dist.destroy_process_group()


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=120))
    from naju_b200.sharded import naju_scan_time_sharded
    B, T, D, N = 2, 400, 160, 16
    d = oracle.make_inputs(B, T, D, N, seed=4, f_shift=3.0, d_skip_scale=0.01, with_h0=True)
    lo, hi = rank * T // world, (rank + 1) * T // world
    dev = torch.device("cuda", rank)
    t = {k: torch.tensor(d[k][:, lo:hi], device=dev).requires_grad_(True) for k in ("u", "fl", "il", "Bm", "Cm")}
    Dk = torch.tensor(d["Dskip"], device=dev).requires_grad_(True)
    h0 = torch.tensor(d["h0"], device=dev).requires_grad_(True) if rank == 0 else None
    y, h_end, _ = naju_scan_time_sharded(t["u"], t["fl"], t["il"], t["Bm"], t["Cm"], Dk, None, h0=h0,
                                         return_final_state=True)
    outs, grads = [y], [torch.tensor(d["dy"][:, lo:hi], device=dev)]
    if rank == world - 1:
        outs.append(h_end)
        grads.append(torch.tensor(d["dhT"], device=dev))
    torch.autograd.backward(outs, grads)
    with torch.no_grad():   # inference route: carry fix-up on the leading part only
        y_ng = naju_scan_time_sharded(t["u"].detach(), t["fl"].detach(), t["il"].detach(), t["Bm"].detach(),
                                      t["Cm"].detach(), Dk.detach(), None, h0=None if h0 is None else h0.detach())
    res = dict(rank=rank, y=y.detach().cpu().numpy(), y_ng=y_ng.cpu().numpy(), h_end=h_end.detach().cpu().numpy(),
               dD=Dk.grad.cpu().numpy(), **{"d" + k: t[k].grad.cpu().numpy() for k in t})
    if rank == 0:
        res["dh0"] = h0.grad.cpu().numpy()
    q.put(res)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_nccl_hand_off_matches_unsharded_oracle(world):
    """Time-sharded scan over `world` ranks, one process per GPU, NCCL hand-off of (state, decay)
    (NVLS off, plain send/recv), forward and backward against the unsharded fp64 oracle."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=300) for _ in range(world)], key=lambda r: r["rank"])
    for p in procs:
        p.join(60)
    B, T, D, N = 2, 400, 160, 16
    d = oracle.make_inputs(B, T, D, N, seed=4, f_shift=3.0, d_skip_scale=0.01, with_h0=True)
    a = (d["u"], d["fl"], d["il"], d["Bm"], d["Cm"], d["Dskip"])
    y, hT = oracle.oracle_fwd(*a, h0=d["h0"], return_final_state=True)
    g = oracle.oracle_bwd(*a, d["dy"], h0=d["h0"], dhT=d["dhT"])
    cat = lambda k: np.concatenate([r[k] for r in res], axis=1)
    assert oracle.rel_l2(cat("y"), y) < 2e-5
    assert oracle.rel_l2(cat("y_ng"), y) < 2e-5
    assert oracle.rel_l2(res[-1]["h_end"], hT) < 2e-5
    for k, gk in (("du", "du"), ("dfl", "dfl"), ("dil", "dil"), ("dBm", "dB"), ("dCm", "dC")):
        assert oracle.rel_l2(cat(k), g[gk]) < 1e-4, k
    assert oracle.rel_l2(sum(r["dD"] for r in res), g["dD"]) < 1e-4
    assert oracle.rel_l2(res[0]["dh0"], g["dh0"]) < 1e-4


def _worker_channels(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=120))
    from naju_b200.sharded import naju_scan_channel_sharded, shard_channels
    B, T, D, N = 2, 400, 384, 16
    d = oracle.make_inputs(B, T, D, N, seed=7, f_shift=2.0, d_skip_scale=0.01, with_h0=True)
    dev = torch.device("cuda", rank)
    # the slices are views with the full tensor's row stride: they go to the kernels without a copy
    sl = lambda a, dim: shard_channels(torch.tensor(a, device=dev), rank, world, dim=dim)
    t = {k: sl(d[k], 2).requires_grad_(True) for k in ("u", "fl", "il")}
    t["Bm"], t["Cm"] = (torch.tensor(d[k], device=dev).requires_grad_(True) for k in ("Bm", "Cm"))
    Dk = sl(d["Dskip"], 0).requires_grad_(True)
    h0 = sl(d["h0"], 1).requires_grad_(True)
    y, hT = naju_scan_channel_sharded(t["u"], t["fl"], t["il"], t["Bm"], t["Cm"], Dk, None, h0=h0,
                                      return_final_state=True)
    torch.autograd.backward([y, hT], [sl(d["dy"], 2), sl(d["dhT"], 1)])
    q.put(dict(rank=rank, y=y.detach().cpu().numpy(), hT=hT.detach().cpu().numpy(), dD=Dk.grad.cpu().numpy(),
               dh0=h0.grad.cpu().numpy(), **{"d" + k: t[k].grad.cpu().numpy() for k in t}))
    dist.barrier()
    dist.destroy_process_group()


def test_nccl_channel_sharded_matches_unsharded_oracle():
    """Channel slices on two GPUs (B and C replicated, no exchange in the forward), dB and dC
    completed by one NCCL all-reduce (NVLS off); fp32 against the unsharded fp64 oracle."""
    world = 2
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_channels, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=300) for _ in range(world)], key=lambda r: r["rank"])
    for p in procs:
        p.join(60)
    B, T, D, N = 2, 400, 384, 16
    d = oracle.make_inputs(B, T, D, N, seed=7, f_shift=2.0, d_skip_scale=0.01, with_h0=True)
    a = (d["u"], d["fl"], d["il"], d["Bm"], d["Cm"], d["Dskip"])
    y, hT = oracle.oracle_fwd(*a, h0=d["h0"], return_final_state=True)
    g = oracle.oracle_bwd(*a, d["dy"], h0=d["h0"], dhT=d["dhT"])
    cat = lambda k, ax: np.concatenate([r[k] for r in res], axis=ax)
    assert oracle.rel_l2(cat("y", 2), y) < 2e-5
    assert oracle.rel_l2(cat("hT", 1), hT) < 2e-5
    for k, gk in (("du", "du"), ("dfl", "dfl"), ("dil", "dil")):
        assert oracle.rel_l2(cat(k, 2), g[gk]) < 1e-4, k
    assert oracle.rel_l2(cat("dD", 0), g["dD"]) < 1e-4
    assert oracle.rel_l2(cat("dh0", 1), g["dh0"]) < 1e-4
    for r in res:
        assert oracle.rel_l2(r["dBm"], g["dB"]) < 1e-4
        assert oracle.rel_l2(r["dCm"], g["dC"]) < 1e-4
