#!/usr/bin/env python
"""Benchmark of the gated-scan hot path: forward + backward scan throughput.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (the headline metric's configuration): B=8, T=16384, D=2048, N=16, bf16 inputs, fp32 state,
synthetic seeded inputs u~N(0,1), f_logit~N(2,1), i_logit~N(0,1), B,C~N(0,1/N), dy~N(0,1).
A step is one forward + one backward scan over that batch.  With N>1 GPUs every rank runs
the same batch shape on its own data (batch sharding, no collective): weak scaling.

Prints ONE JSON line on rank 0.  `value` is tokens/s with inputs resident in HBM; `e2e`
is the same metric through the public `naju_scan` call with HOST buffers, host<->device
copies inside the timed region.  `--impl reference` times the CPU restatement of the
reference scan (oracle/) on the host cores instead.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def host_threads():
    """Host threads this process may use (its CPU affinity, not the machine's core count)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


# The CPU legs use every host thread.  torch.distributed.run exports OMP_NUM_THREADS=1 to its
# workers, which would silently time the OpenMP oracle on one core: set the count explicitly,
# before any OpenMP runtime is loaded.
os.environ["OMP_NUM_THREADS"] = str(host_threads())

METRIC = "scan fwd+bwd tokens/sec and HBM GB/s % of peak, B=8 L=16K D=2048 N=16"
CFG = dict(B=8, T=16384, D=2048, N=16)
FALLBACK_HBM_GBS = 6650.0


def algorithmic_bytes(B, T, D, N, e=2, eg=None):
    """Per-launch algorithmic HBM bytes: forward reads u,fl,il,B,C and writes y;
    backward reads u,fl,il,dy,B,C and writes du,dfl,dil,dB,dC.  e = element size of the
    activations, eg = of the logits and their gradients (e unless given)."""
    tok = B * T
    eg = e if eg is None else eg
    return tok * (2 * D * e + 2 * D * eg + 2 * N * e), tok * (3 * D * e + 4 * D * eg + 4 * N * e)


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.path = index, None, f"/tmp/naju_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "100"], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        for line in open(self.path):
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1])); mx.append(float(c[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                "sw_power_cap"), c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.remove(self.path)
        except OSError:
            pass
        if sm:
            # samples under load: the upper half of the sampled clocks
            out["sm_mhz"] = statistics.median(sm)
            out["sm_max_mhz"] = max(mx)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


# ----------------------------------------------------------------------------- CPU arm
def cpu_reference_run(steps, warmup, target_s=2.5):
    """Times the CPU restatement of the reference scan (forward + backward, fp32) on all host
    threads.  One step is a bounded sample of the metric workload: B=1, D=2048, N=16 and a
    time length chosen so that a step takes about `target_s` seconds."""
    import oracle
    D, N = CFG["D"], CFG["N"]
    cores = oracle.oracle_threads()

    def one(T, seed=0):
        d = oracle.make_inputs(1, T, D, N, seed=seed)
        a = (d["u"], d["fl"], d["il"], d["Bm"], d["Cm"], d["Dskip"])
        t0 = time.perf_counter()
        oracle.oracle_fwd(*a, precision="f32")
        oracle.oracle_bwd(*a, d["dy"], precision="f32")
        return time.perf_counter() - t0

    t_probe = one(64)
    T = int(min(65536, max(64, 64 * target_s / max(t_probe, 1e-4))))
    for _ in range(warmup):
        one(T)
    times = [one(T) for _ in range(steps)]
    ms = 1e3 * sum(times) / len(times)
    value = T / (ms / 1e3)
    sample = f"B=1,T={T},D={D},N={N} fp32, {steps} steps after {warmup} warm-up"
    return value, ms, cores, sample


def reference_python_run():
    """The reference's own `naju_scan_reference` (naju/scan.py:79-93) forward + autograd backward at
    its CPU-runnable configuration (B=2, T=512, D=64, N=16, fp32, seed 0): median of 5 after one
    warm-up, all host threads.  Only where the reference tree can be imported (NAJU_REFERENCE_PATH);
    returns None elsewhere."""
    path = os.environ.get("NAJU_REFERENCE_PATH")
    if not path or not os.path.isdir(os.path.join(path, "naju")):
        return None
    import torch
    sys.path.insert(0, path)
    try:
        from naju.scan import naju_scan_reference
    except Exception:
        return None
    finally:
        sys.path.remove(path)
    torch.set_num_threads(host_threads())
    B, T, D, N = 2, 512, 64, 16
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g)
    u, fl, il = r(B, T, D), r(B, T, D) + 2.0, r(B, T, D)
    Bm, Cm, dy = r(B, T, N) / N ** 0.5, r(B, T, N) / N ** 0.5, r(B, T, D)
    leaves = [t.requires_grad_(True) for t in (u, fl, il, Bm, Cm)]
    times = []
    for k in range(6):
        for t in leaves:
            t.grad = None
        t0 = time.perf_counter()
        naju_scan_reference(*leaves, torch.zeros(D)).backward(dy)
        times.append(time.perf_counter() - t0)
    med = statistics.median(times[1:])
    return {"value": B * T / med, "unit": "tokens/s", "cores": torch.get_num_threads(),
            "sample": "naju_scan_reference fwd+bwd, B=2,T=512,D=64,N=16 fp32, median of 5 after 1 warm-up",
            "torch": torch.__version__}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    value, ms, cores, sample = cpu_reference_run(args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "metric: scan fwd+bwd B=8 T=16384 D=2048 N=16 (bounded CPU sample)",
                   "sample": sample},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    ref_py = reference_python_run()
    if ref_py is not None:
        line["cpu_baseline"]["reference_python"] = ref_py
    print(json.dumps(line), flush=True)


def ncu_traffic_bwd(B, T, D, N):
    """DRAM bytes of one tensor-core backward launch, scaled from the ncu capture recorded in
    profiles/dram_traffic_per_token.txt (JSON: bytes per token of the captured small case, keyed
    by "D,N").  Traffic grows in proportion to the tokens (every tile moves the same bytes), so a
    full launch is that figure times the token count.  None when no capture covers the shape."""
    try:
        rec = json.load(open(os.path.join(ROOT, "profiles", "dram_traffic_per_token.txt")))
        return float(rec["bwd_tc_kernel"][f"{D},{N}"]) * (B * T)
    except Exception:
        return None


# ----------------------------------------------------------------------------- GPU arm
def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    from naju_b200 import naju_scan

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (there is no CPU fallback for the scan)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    B, T, D, N = args.shape
    dt = torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(rank)

    def rn(*s):
        return torch.randn(*s, device=dev, generator=g)

    u = rn(B, T, D).to(dt)
    if args.layout == "mixer":
        # as the mixer hands the tensors over under bf16 autocast (naju/mixer.py:106-118): u is the
        # depthwise convolution's [B,D,T] output viewed as [B,T,D]; the logits are fp32
        u = u.transpose(1, 2).contiguous().transpose(1, 2)
    gdt = torch.float32 if args.layout == "mixer" else dt
    fl = (rn(B, T, D) + 2.0).to(gdt)
    il = rn(B, T, D).to(gdt)
    Bm = (rn(B, T, N) / N ** 0.5).to(dt)
    Cm = (rn(B, T, N) / N ** 0.5).to(dt)
    Dk = torch.zeros(D, device=dev)
    dy = rn(B, T, D).to(dt)
    leaves = [u, fl, il, Bm, Cm, Dk]
    for t in leaves:
        t.requires_grad_(True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step(ev=None):
        for t in leaves:
            t.grad = None
        if ev:
            ev[0].record()
        y = naju_scan(u, fl, il, Bm, Cm, Dk)
        if ev:
            ev[1].record()
        y.backward(dy)
        if ev:
            ev[2].record()
        return y

    for _ in range(args.warmup):
        step()
    barrier()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    t_begin = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    barrier()
    t_begin.record()
    for k in range(args.steps):
        step(evs[k])
    t_end.record()
    barrier()
    total_ms = t_begin.elapsed_time(t_end)
    fwd_ms = sum(e[0].elapsed_time(e[1]) for e in evs) / args.steps
    bwd_ms = sum(e[1].elapsed_time(e[2]) for e in evs) / args.steps
    # The reference's own protocol (naju/tests/bench_scan.py:39-54) is the median of >= 30 iterations
    # after >= 10 warm-ups: by now at least 3 + K steps have run; time 30 more, each on its own events,
    # and report their median beside the K-step mean.
    evm = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(max(30, args.steps))]
    for _ in range(max(0, 10 - args.warmup - args.steps)):
        step()
    for e in evm:
        step(e)
    barrier()
    med = {"median_ms_per_step": statistics.median(e[0].elapsed_time(e[2]) for e in evm),
           "median_fwd_ms": statistics.median(e[0].elapsed_time(e[1]) for e in evm),
           "median_bwd_ms": statistics.median(e[1].elapsed_time(e[2]) for e in evm),
           "median_over_steps": len(evm)}

    # ---- end to end through the public call with HOST buffers
    if args.no_e2e:
        return _finish(args, world, rank, dev, dist, torch, total_ms, None, fwd_ms, bwd_ms,
                       sampler, 0, 0, 0, med)
    # Inputs live in pinned host memory; the call streams batch rows through the GPU (copy in,
    # forward + backward, copy out on three streams) and leaves y and every gradient in pinned
    # host memory.  All of that is inside the timed region.
    from naju_b200 import scan_fwd_bwd_host
    host_in = [t.detach().cpu().pin_memory() for t in (u, fl, il, Bm, Cm, dy)]
    Dk_host = Dk.detach().cpu()
    h2d = sum(t.numel() * t.element_size() for t in host_in) + Dk_host.numel() * 4
    host_out = None
    e2e_steps = max(1, min(args.steps, 5))

    def e2e_step():
        nonlocal host_out
        host_out = scan_fwd_bwd_host(host_in[0], host_in[1], host_in[2], host_in[3], host_in[4], Dk_host,
                                     host_in[5], rows_per_chunk=1, time_splits=2, out=host_out)
        return host_out

    e2e_step()
    barrier()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    d2h = sum(t.numel() * t.element_size() for t in host_out.values())
    return _finish(args, world, rank, dev, dist, torch, total_ms, e2e_ms, fwd_ms, bwd_ms, sampler,
                   h2d, d2h, e2e_steps, med)


def _finish(args, world, rank, dev, dist, torch, total_ms, e2e_ms, fwd_ms, bwd_ms, sampler, h2d,
            d2h, e2e_steps, med):
    B, T, D, N = args.shape
    clocks = sampler.stop() if rank == 0 else None
    times = torch.tensor([total_ms, e2e_ms or 0.0, fwd_ms, bwd_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, fwd_ms, bwd_ms = times.tolist()

    if rank == 0:
        tokens = B * T * world
        ms_per_step = total_ms / args.steps
        value = tokens / (ms_per_step / 1e3)
        fwd_bytes, bwd_bytes = algorithmic_bytes(B, T, D, N, eg=4 if args.layout == "mixer" else 2)
        peak, peak_kind = measured_peak()
        achieved = bwd_bytes / (bwd_ms / 1e3) / 1e9
        is_metric = (B, T, D, N) == (CFG["B"], CFG["T"], CFG["D"], CFG["N"])
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": ("metric: " if is_metric else "other: ") +
                       f"scan fwd+bwd B={B} T={T} D={D} N={N} per GPU",
                       "io_dtype": "bf16" if args.layout == "reference" else
                       "bf16 u/B/C, fp32 logits; u time-contiguous ([B,D,T] memory), as naju/mixer.py hands them over",
                       "state_dtype": "f32", "sharding": f"batch x{world}, no collective",
                       "l2": "inputs larger than L2 (no flush needed)",
                       "d_skip": "zeros, as the mixer passes them (the skip is applied outside the scan)",
                       "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
                       "fwd_gbs": fwd_bytes / (fwd_ms / 1e3) / 1e9,
                       "fwd_bwd_gbs": (fwd_bytes + bwd_bytes) / (ms_per_step / 1e3) / 1e9,
                       "fwd_bwd_frac_of_peak": (fwd_bytes + bwd_bytes) / (ms_per_step / 1e3) / 1e9 / peak,
                       **med},
            "roofline": {"bound": "hbm", "kernel": "bwd_tc_kernel", "achieved": achieved,
                         "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": ncu_traffic_bwd(B, T, D, N),
                         "algorithmic_bytes_per_launch": bwd_bytes},
            # forward, tensor-core backward, recurrent backward (stands down), 3 finalize kernels, and
            # the failure check after the forward and after the backward
            "gpu_launches": 8 * args.steps,
            "clocks": clocks,
        }
        if e2e_steps:
            line["e2e"] = {"value": B * T * world / (e2e_ms / 1e3), "unit": "tokens/s",
                           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                           "ms_per_step": e2e_ms, "steps": e2e_steps,
                           "call": "naju_b200.scan_fwd_bwd_host (pinned host tensors in and out, one batch "
                                   "row per chunk in two time segments, copies overlapped with the kernels)"}
        if world == 1 and not args.no_cpu_baseline:
            v, ms, cores, sample = cpu_reference_run(3, 1, target_s=2.0)
            line["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port",
                                    "sample": sample}
            ref_py = reference_python_run()
            if ref_py is not None:
                line["cpu_baseline"]["reference_python"] = ref_py
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_decode(args):
    """Decode-step leg (not the headline): one token for 24 layers of state [256, 2048, 16] fp32,
    each layer's state updated in place by one launch.  24 x 33.5 MB of state (805 MB) is larger
    than L2, so every launch reads and writes its state from HBM: 2*N*4 bytes per channel plus the
    token's u / logits / y."""
    import torch
    from naju_b200 import naju_scan_step
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (there is no CPU fallback for the scan)")
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    L, Bsz, D, N = 24, 256, 2048, 16
    g = torch.Generator(device=dev).manual_seed(3)
    states = [torch.randn(Bsz, D, N, device=dev, generator=g) for _ in range(L)]
    bf = torch.bfloat16
    u = torch.randn(Bsz, D, device=dev, generator=g).to(bf)
    fl = (torch.randn(Bsz, D, device=dev, generator=g) + 2).to(bf)
    il = torch.randn(Bsz, D, device=dev, generator=g).to(bf)
    Bm = (torch.randn(Bsz, N, device=dev, generator=g) / 4).to(bf)
    Cm = (torch.randn(Bsz, N, device=dev, generator=g) / 4).to(bf)
    Dk = torch.zeros(D, device=dev)

    def step():
        for st in states:
            naju_scan_step(st, u, fl, il, Bm, Cm, Dk)

    def timed(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.steps

    eager_ms = timed(step)
    # the 24 launches of one token captured once in a CUDA graph and replayed (no per-launch host work)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    ms = timed(graph.replay)
    nbytes = L * (2 * Bsz * D * N * 4 + Bsz * D * 2 * 4)
    peak, peak_kind = measured_peak()
    gbs = nbytes / (ms / 1e3) / 1e9
    print(json.dumps({
        "metric": "decode state update, 24 layers x batch 256 x D=2048 x N=16", "value": Bsz / (ms / 1e3),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
        "higher_is_better": True, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "decode: 24 launches of step_kernel per token (one CUDA graph replay), state in place",
                   "eager_ms_per_step": eager_ms},
        "roofline": {"bound": "hbm", "kernel": "step_kernel", "achieved": gbs, "peak": peak,
                     "peak_kind": peak_kind, "unit": "GB/s", "frac": gbs / peak, "traffic": None,
                     "algorithmic_bytes_per_launch": nbytes // L},
        "gpu_launches": L * args.steps}), flush=True)


def run_layer(args):
    """Whole-layer leg (not the headline): the computation of one Naju mixer layer at config 1's
    size (d_model 1024, expand 2, d_state 16, batch 8, 4096 tokens, bf16 autocast, weights
    N(0, 0.02^2)), forward + backward, with this library's scan in the place naju/mixer.py:121-122
    calls `naju_scan`.  The layer is restated here with torch functional ops in the order of
    naju/mixer.py:112-125 (the reference's module itself is not on this machine); everything but the
    scan is cuBLAS / cuDNN / torch elementwise, as in the reference.  Reports the layer's time and
    the scan's share of it."""
    import torch
    import torch.nn.functional as F
    from naju_b200 import naju_scan
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (there is no CPU fallback for the scan)")
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    Bsz, T, d_model, N, K = 8, 4096, 1024, 16, 4
    D = 2 * d_model
    g = torch.Generator(device=dev).manual_seed(1)

    def w(*shape):
        return (torch.randn(*shape, device=dev, generator=g) * 0.02).requires_grad_(True)

    W_in, W_x, W_f, W_i, W_out = w(2 * D, d_model), w(2 * N, D), w(D, D), w(D, D), w(d_model, D)
    cw, fw, iw = w(D, 1, K), w(D, 1, K), w(D, 1, K)
    cb = torch.zeros(D, device=dev, requires_grad=True)
    f_bias = torch.full((D,), 5.0, device=dev, requires_grad=True)
    i_bias = torch.full((D,), -2.0, device=dev, requires_grad=True)
    Dp = torch.full((D,), 0.01, device=dev, requires_grad=True)
    D_zero = torch.zeros(D, device=dev)
    params = [W_in, W_x, W_f, W_i, W_out, cw, fw, iw, cb, f_bias, i_bias, Dp]
    hidden = torch.randn(Bsz, T, d_model, device=dev, generator=g).requires_grad_(True)
    dout = torch.randn(Bsz, T, d_model, device=dev, generator=g).to(torch.bfloat16)
    ev = {}

    def layer(timed_scan):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            x, z = F.linear(hidden, W_in).chunk(2, dim=-1)
            x = F.silu(F.conv1d(x.transpose(1, 2), cw, cb, padding=K - 1, groups=D)[..., :T].transpose(1, 2))
            Bm, Cm = torch.split(F.linear(x, W_x), [N, N], dim=-1)
            xt = x.transpose(1, 2)
            fl = F.linear(x, W_f) + F.conv1d(xt, fw, None, padding=K - 1, groups=D)[..., :T].transpose(1, 2) + f_bias
            il = F.linear(x, W_i) + F.conv1d(xt, iw, None, padding=K - 1, groups=D)[..., :T].transpose(1, 2) + i_bias
            if timed_scan:
                ev["f0"].record()
            cx = naju_scan(x, fl, il, Bm, Cm, D_zero)
            if timed_scan:
                ev["f1"].record()
            y = (cx * (1.0 / N ** 0.5) + Dp * x) * F.silu(z)
            out = F.linear(y, W_out)
        return out

    def step(timed_scan=False):
        for p in params + [hidden]:
            p.grad = None
        out = layer(timed_scan)
        out.backward(dout)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    steps = max(args.steps, 5)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    layer_ms = e0.elapsed_time(e1) / steps
    # the scan alone, on the tensors the layer hands it (same layouts and dtypes), forward + backward
    with torch.autocast("cuda", dtype=torch.bfloat16):
        x, z = F.linear(hidden, W_in).chunk(2, dim=-1)
        x = F.silu(F.conv1d(x.transpose(1, 2), cw, cb, padding=K - 1, groups=D)[..., :T].transpose(1, 2))
        Bm, Cm = torch.split(F.linear(x, W_x), [N, N], dim=-1)
        fl = F.linear(x, W_f) + f_bias
        il = F.linear(x, W_i) + i_bias
    leaves = [t.detach().clone(memory_format=torch.preserve_format).requires_grad_(True) for t in (x, fl, il)]
    bc = torch.cat([Bm, Cm], -1).detach().requires_grad_(True)
    Bv, Cv = torch.split(bc, [N, N], dim=-1)
    dy = torch.randn(Bsz, T, D, device=dev, generator=g).to(torch.bfloat16)
    ts = []
    for k in range(steps + 3):
        for p in leaves + [bc]:
            p.grad = None
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        naju_scan(leaves[0], leaves[1], leaves[2], Bv, Cv, D_zero).backward(dy)
        b.record()
        torch.cuda.synchronize()
        if k >= 3:
            ts.append(a.elapsed_time(b))
    scan_ms = sum(ts) / len(ts)
    print(json.dumps({
        "metric": "one mixer layer fwd+bwd, d_model 1024, expand 2, N=16, batch 8 x 4096 tokens, bf16 autocast",
        "value": Bsz * T / (layer_ms / 1e3), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": max(args.warmup, 3), "ms_per_step": layer_ms, "higher_is_better": True, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": "layer: the ops of naju/mixer.py:112-125 restated with torch functional calls, "
                               "this library's scan in place of naju_scan",
                   "scan_fwd_bwd_ms": scan_ms, "scan_share": scan_ms / layer_ms,
                   "u_layout": list(leaves[0].stride()), "logit_dtype": str(leaves[1].dtype)},
        "gpu_launches": 8 * steps}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--shape", default=None, help="B,T,D,N instead of the metric workload (profiling)")
    ap.add_argument("--layout", default="reference", choices=["reference", "mixer"],
                    help="reference = contiguous bf16 [B,T,D] tensors (the metric); mixer = u in [B,D,T] memory "
                         "and fp32 logits, as the mixer produces them (a side measurement, not the metric)")
    ap.add_argument("--workload", default="train", choices=["train", "decode", "layer"],
                    help="train = the headline fwd+bwd scan; decode = the single-token state update; "
                         "layer = one mixer layer at config 1's size with the scan's share of its time")
    args = ap.parse_args()
    args.shape = tuple(int(x) for x in args.shape.split(",")) if args.shape else \
        (CFG["B"], CFG["T"], CFG["D"], CFG["N"])
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "decode":
        run_decode(args)
    elif args.workload == "layer":
        run_layer(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
