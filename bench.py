#!/usr/bin/env python
"""Benchmark of the oriented 1D depthwise convolution on B200.

Workload ("stage sweep"): the operator at the four ConvNeXt-T stage shapes
(H=W, C) = (56,96), (28,192), (14,384), (7,768), batch 128 per GPU, K=31, stride 1,
NHWC, 8 orientations assigned round-robin, fp32, synthetic N(0,1) inputs.  One step runs
fprop, dgrad and wgrad once at each shape (12 operator calls).  Throughput is images/s:
128 images x GPUs per step.

    python bench.py [--gpus N] [--steps K] [--warmup W]      # this implementation
    python bench.py --impl reference ...                      # the reference's CPU operator

Prints ONE JSON line.  Extra keys: `kernels` (per-kernel time, algorithmic GB/s and
fraction of the measured HBM copy rate, fp32 and bf16, round-robin angles; `tr_*` are the
layout transposes), `kernels_block` (the same with the models' block-wise angle assignment),
`roofline` (the kernel that takes the most time), `cpu_baseline`, `cpu_conv2d` (the operator as
a torch depthwise conv2d over the rasterised kernel on all host cores), `e2e` (same work
through the nn.Module with host buffers: H2D of inputs and D2H of all results inside the timed
region), `model` (ConvNeXt-T-1D inference img/s on the same GPUs), `clocks`.

Other workloads, one JSON line each: `--workload model` (ConvNeXt-T-1D inference, bf16, batch
256 per GPU), `--workload train` (ConvNeXt-B-1D++ training step: cross-entropy, AdamW, one flat
all-reduce of every gradient), `--workload dense` (dense-prediction backbone, forward + backward
at 800x1280).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

STAGES = [(56, 96), (28, 192), (14, 384), (7, 768)]
BATCH = 128
K = 31
L2_BYTES = 126 * 1024 * 1024
METRIC = "dwoconv1d stage-sweep throughput (fprop+dgrad+wgrad at the 4 ConvNeXt-T stage shapes)"
HBM_FALLBACK_GBS = 6650.0


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return HBM_FALLBACK_GBS, "fallback"


def round_robin_angles(C, n=8):
    """theta[c] = (c mod n) * pi / n as fp32: the sweep's channel -> orientation assignment."""
    import numpy as np
    return np.array([(c % n) * np.pi / n for c in range(C)], dtype=np.float64).astype(np.float32)


def block_angles(C, n=8):
    """The models' assignment: blocks of ~C/n consecutive channels share an angle
    (reference: models/convnext.py:60-65)."""
    import numpy as np
    return np.array([((n * (c + 1) - 1) // C) * np.pi / n for c in range(C)], dtype=np.float64).astype(np.float32)


def algorithmic_bytes(hw, C, esize, n=BATCH):
    """One tensor in, one tensor out (or two in for wgrad) plus the fp32 taps."""
    return 2 * n * hw * hw * C * esize + C * K * 4


# --------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except Exception:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


# --------------------------------------------------------------------------------------
# reference arm / cpu baseline: the reference's own CPU loops (oracle/_ref), else the port
# --------------------------------------------------------------------------------------
def cpu_loops():
    from oracle.oracle import Oracle, Reference
    if Reference.available():
        return Reference(), "reference"
    return Oracle(), "port"


def host_threads():
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_step(loops, n_img, seed=0, threads=1):
    """fprop + dgrad + wgrad at the four stage shapes on n_img images; returns seconds.

    The loops are single-threaded as written (kernels.cpp:36-52, :71-90, :111-126).  With
    threads > 1 the batch is cut into per-thread slices and the same unmodified loops run on the
    slices concurrently (ctypes releases the GIL); fprop and dgrad are independent per image and
    the per-slice weight gradients are added at the end, inside the timed region."""
    import numpy as np
    from oracle.oracle import round_robin_angles
    rng = np.random.default_rng(seed)
    total = 0.0
    pool = None
    if threads > 1:
        from concurrent.futures import ThreadPoolExecutor
        pool = ThreadPoolExecutor(threads)
    bounds = [(i * n_img // threads, (i + 1) * n_img // threads) for i in range(threads)]
    bounds = [(lo, hi) for lo, hi in bounds if hi > lo]
    for hw, C in STAGES:
        x = rng.standard_normal((n_img, C, hw, hw)).astype(np.float32)
        dy = rng.standard_normal((n_img, C, hw, hw)).astype(np.float32)
        w = (0.02 * rng.standard_normal((C, 1, 1, K))).astype(np.float32)
        th = round_robin_angles(C)

        def work(b, x=x, dy=dy, w=w, th=th):
            xs, dys = np.ascontiguousarray(x[b[0]:b[1]]), np.ascontiguousarray(dy[b[0]:b[1]])
            loops.fprop(xs, w, th, 1)
            loops.dgrad(dys, w, th, 1)
            return loops.wgrad(dys, xs, th, K, 1)

        t0 = time.perf_counter()
        if pool is None:
            work((0, n_img))
        else:
            sum(pool.map(work, bounds))
        total += time.perf_counter() - t0
    if pool is not None:
        pool.shutdown()
    return total


def cpu_conv2d_baseline():
    """The operator as the reference's CPU formulation: torch depthwise conv2d over the (2 pad + 1)^2
    kernel that has w[c, k] scatter-added at tap k's rasterised offset; forward plus autograd
    backward (input and weight gradients) on all host cores, at N=2, 56x56x96, K=31, round-robin
    angles (the single-layer CPU configuration)."""
    import numpy as np
    import torch
    import torch.nn.functional as F
    from oracle.oracle import Oracle
    N, C, hw, pad = 2, 96, 56, K // 2
    g = torch.Generator().manual_seed(0)
    x = torch.randn((N, C, hw, hw), generator=g, requires_grad=True)
    w = (0.02 * torch.randn((C, K), generator=g)).requires_grad_(True)
    dy = torch.randn((N, C, hw, hw), generator=g)
    dh, dw = Oracle().offsets(round_robin_angles(C), K)
    ci = torch.arange(C).repeat_interleave(K)
    ri = torch.from_numpy(np.ascontiguousarray(dh, np.int64)).reshape(-1) + pad
    qi = torch.from_numpy(np.ascontiguousarray(dw, np.int64)).reshape(-1) + pad

    def fwd():
        k2d = torch.zeros((C, 1, 2 * pad + 1, 2 * pad + 1)).index_put((ci, torch.zeros_like(ci), ri, qi),
                                                                     w.reshape(-1), accumulate=True)
        return F.conv2d(x, k2d, None, 1, pad, 1, C)

    fwd().backward(dy)                       # warm-up
    reps, tf, tb = 3, 0.0, 0.0
    for _ in range(reps):
        x.grad = w.grad = None
        t0 = time.perf_counter()
        y = fwd()
        t1 = time.perf_counter()
        y.backward(dy)
        t2 = time.perf_counter()
        tf, tb = tf + t1 - t0, tb + t2 - t1
    return {"value": N * reps / (tf + tb), "unit": "img/s", "cores": torch.get_num_threads(), "kind": "port",
            "forward_s": tf / reps, "backward_s": tb / reps,
            "sample": f"N={N}, 56x56x96, K=31, fp32 NCHW, forward + backward, {reps} repetitions: "
                      "F.conv2d(groups=C) over the scatter-added 31x31 kernel"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    torch.set_num_threads(1)              # the slices are the parallelism
    loops, kind = cpu_loops()
    threads = host_threads()
    n_img = 4 * threads
    for _ in range(args.warmup):
        cpu_step(loops, n_img, threads=threads)
    t = sum(cpu_step(loops, n_img, seed=i, threads=threads) for i in range(args.steps))
    value = n_img * args.steps / t
    sample = (f"{n_img} images per step at each of the 4 stage shapes, fp32 NCHW, the reference's single-threaded "
              f"loops on {threads} batch slices in {threads} threads")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "img/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "stage-sweep: (56,96),(28,192),(14,384),(7,768) x batch 128, K=31, stride 1, "
                               "8 orientations round-robin; fprop+dgrad+wgrad per shape",
                   "sample_images_per_step": n_img},
        "cpu_baseline": {"value": value, "unit": "img/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "img/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------------------
# this implementation
# --------------------------------------------------------------------------------------
def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    import oriented1d_b200 as o1d

    world, rank, local, dev = init_ranks()

    peak, peak_src = measured_peak()
    g = torch.Generator(device="cpu").manual_seed(rank)

    class Layer:
        """One stage shape: rotating input sets so that successive launches never find
        their inputs in L2 (each set is touched once per `nsets` launches and the sets
        together exceed 4x the L2 size)."""

        def __init__(self, hw, C, dtype, angles=round_robin_angles):
            self.hw, self.C, self.dtype = hw, C, dtype
            es = 4 if dtype == torch.float32 else 2
            per_set = 2 * BATCH * hw * hw * C * es
            self.nsets = max(2, -(-4 * L2_BYTES // per_set))
            self.plan = o1d.Plan(angles(C), K)
            self.w = (0.02 * torch.randn((C, 1, 1, K), generator=g)).to(dev)
            base_x = torch.randn((BATCH, hw, hw, C), generator=g)
            base_dy = torch.randn((BATCH, hw, hw, C), generator=g)
            self.x = [base_x.to(dev).to(dtype).clone() for _ in range(self.nsets)]
            self.dy = [base_dy.to(dev).to(dtype).clone() for _ in range(self.nsets)]
            self.i = 0

        def next(self):
            self.i = (self.i + 1) % self.nsets
            return self.x[self.i], self.dy[self.i]

    layers32 = [Layer(hw, C, torch.float32) for hw, C in STAGES]
    launches = {"n": 0}

    def compute(layers):
        """The 12 kernel calls of one step; returns the weight/bias gradients as one flat buffer."""
        grads = []
        for L in layers:
            x, dy = L.next()
            o1d.fprop(x, L.w, None, L.plan, 1, True)
            o1d.dgrad(dy, L.w, L.plan, L.hw, L.hw, 1, True)
            dw, db = o1d.wgrad(dy, x, L.plan, 1, True, True)
            grads += [dw.reshape(-1), db]
            launches["n"] += o1d.ops.KERNELS_PER_CALL["fprop"] + o1d.ops.KERNELS_PER_CALL["dgrad"] + \
                o1d.ops.KERNELS_PER_CALL["wgrad"]
        return torch.cat(grads) if world > 1 else None

    def step(layers):
        flat = compute(layers)
        if world > 1:   # data-parallel training sums the weight gradients across ranks
            dist.all_reduce(flat)

    comm = torch.cuda.Stream(device=dev) if world > 1 else None

    def graphed_multi_gpu_step(layers, cycle):
        """world > 1: one CUDA graph per step of the input rotation (kernels only).  The NCCL
        all-reduce of a step's gradient buffer runs on its own stream under the next step's
        kernels; a graph is replayed again only after the all-reduce that read its buffer."""
        for _ in range(3):
            step(layers)
        torch.cuda.synchronize()
        graphs = []
        for _ in range(cycle):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                flat = compute(layers)
            graphs.append((g, flat, torch.cuda.Event()))
        state = {"i": 0}

        def run():
            cur = torch.cuda.current_stream()
            g, flat, reduced = graphs[state["i"] % cycle]
            state["i"] += 1
            cur.wait_event(reduced)             # the previous all-reduce of this buffer
            g.replay()
            comm.wait_stream(cur)
            with torch.cuda.stream(comm):
                dist.all_reduce(flat)
                reduced.record(comm)
        return run

    def timed(fn, steps, warmup, graph_cycle=0, all_ranks=True, tail=None):
        """Device time of `steps` calls of fn (CUDA events on the launching stream, barrier and
        synchronize on both sides, max over ranks).  `tail` runs after the last call, inside the
        timed region (joins work the calls left on other streams).  With graph_cycle > 0 the calls are captured
        once into a CUDA graph of `graph_cycle` consecutive calls (one full rotation of the input
        sets) and replayed, so that host launch latency does not sit between kernels.
        all_ranks=False: a measurement only this rank takes (no barrier, no max-reduce)."""
        multi = all_ranks and world > 1
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        runner, per = fn, 1
        if graph_cycle > 0:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(graph_cycle):
                    fn()
            graph.replay()                      # one untimed replay
            runner, per = graph.replay, graph_cycle
        reps = max(1, -(-steps // per))
        if multi:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            runner()
        if tail is not None:
            tail()
        e1.record()
        torch.cuda.synchronize()
        if multi:
            dist.barrier()
        ms = e0.elapsed_time(e1) * steps / (reps * per)     # normalised to `steps` calls
        if multi:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    # ---- headline: device-resident inputs --------------------------------------------
    with ClockSampler(local) as clk:
        launches["n"] = 0
        warm = max(args.warmup, 3)
        cycle = max(L.nsets for L in layers32) if (world == 1 and not args.no_graph) else 0
        launches["n"] = 0
        step(layers32)
        per_step = launches["n"]
        if world > 1 and not args.no_graph:
            ms = timed(graphed_multi_gpu_step(layers32, max(L.nsets for L in layers32)), args.steps, warm,
                       tail=lambda: torch.cuda.current_stream().wait_stream(comm))
        else:
            ms = timed(lambda: step(layers32), args.steps, warm, graph_cycle=cycle)
        n_launch = per_step * args.steps
        time.sleep(0.25)
    clocks = clk.summary()
    value = BATCH * world * args.steps / (ms / 1e3)

    # ---- per-kernel timings (rank 0 only, after the headline) -------------------------
    kernels, kernels_block, roof = {}, {}, None
    if rank == 0:
        reps = 40
        for angles, table in ((round_robin_angles, kernels), (block_angles, kernels_block)):
            for dtype, tag in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
                own = not (dtype == torch.float32 and angles is round_robin_angles)
                layers = [Layer(hw, C, dtype, angles) for hw, C in STAGES] if own else layers32
                for L in layers:
                    es = 4 if dtype == torch.float32 else 2
                    ab = algorithmic_bytes(L.hw, L.C, es)

                    def f_fprop(L=L):
                        x, _ = L.next()
                        o1d.fprop(x, L.w, None, L.plan, 1, True)

                    def f_dgrad(L=L):
                        _, dy = L.next()
                        o1d.dgrad(dy, L.w, L.plan, L.hw, L.hw, 1, True)

                    def f_wgrad(L=L):
                        x, dy = L.next()
                        o1d.wgrad(dy, x, L.plan, 1, True, True)

                    def f_tr(L=L):
                        x, _ = L.next()
                        o1d.nhwc_to_nchw(x)

                    cases = [("fprop", f_fprop, ab), ("dgrad", f_dgrad, ab), ("wgrad", f_wgrad, ab)]
                    if angles is round_robin_angles:       # the layout transposes do not depend on the angles
                        cases.append(("tr", f_tr, 2 * BATCH * L.hw * L.hw * L.C * es))
                    for name, fn, nbytes in cases:
                        t_ms = timed(fn, reps, 3, graph_cycle=0 if args.no_graph else L.nsets, all_ranks=False) / reps
                        gbs = nbytes / (t_ms * 1e-3) / 1e9
                        table[f"{name}_{tag}_{L.hw}x{L.hw}x{L.C}"] = {
                            "us": round(t_ms * 1e3, 2), "alg_bytes": nbytes, "gbs": round(gbs, 1),
                            "frac": round(gbs / peak, 4), "route": o1d.ops.last_route() if name != "tr" else None}
                if own:
                    del layers
                    torch.cuda.empty_cache()
        top = max((k for k in kernels if "_f32_" in k and not k.startswith("tr_")), key=lambda k: kernels[k]["us"])
        traffic = None
        try:
            with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
                traffic = json.load(f).get(top)
        except Exception:
            pass
        roof = {"kernel": top, "bound": "hbm", "achieved": kernels[top]["gbs"], "peak": peak, "unit": "GB/s",
                "frac": kernels[top]["frac"], "traffic": traffic, "peak_source": peak_src,
                "alg_bytes_per_launch": kernels[top]["alg_bytes"], "us_per_launch": kernels[top]["us"]}

    # ---- GPU baseline: the reference's own specialised CUDA kernels on this GPU --------
    # (compiled from the reference checkout by oracle/build.py --gpu-reference; NCHW fp32 only;
    # the "nhwc" figure adds the two layout transposes its module wraps around them)
    ref_gpu = None
    if rank == 0 and not args.no_ref_gpu:
        try:
            from oracle.oracle import ReferenceGPU
            refg = ReferenceGPU() if ReferenceGPU.available() else None
        except Exception:
            refg = None
        if refg is not None:
            ref_gpu = {}
            for L in layers32:
                hw, C = L.hw, L.C
                sets = [(x.permute(0, 3, 1, 2).contiguous(), dy.permute(0, 3, 1, 2).contiguous())
                        for x, dy in zip(L.x, L.dy)]
                theta_d = torch.from_numpy(round_robin_angles(C)).to(dev)
                state = {"i": 0}

                def nxt(sets=sets, state=state):
                    state["i"] = (state["i"] + 1) % len(sets)
                    return sets[state["i"]]

                def r_fprop(L=L, theta_d=theta_d):
                    refg.fprop(nxt()[0], L.w, theta_d)

                def r_dgrad(L=L, theta_d=theta_d):
                    refg.dgrad(nxt()[1], L.w, theta_d)

                def r_wgrad(L=L, theta_d=theta_d):
                    x, dy = nxt()
                    refg.wgrad(dy, x, theta_d)

                def r_fprop_nhwc(L=L, theta_d=theta_d, hw=hw, C=C):
                    x = L.next()[0]
                    xc = refg.transpose(x, BATCH, hw * hw, C, (BATCH, C, hw, hw))
                    y = refg.fprop(xc, L.w, theta_d)
                    refg.transpose(y, BATCH, C, hw * hw, (BATCH, hw, hw, C))

                for name, fn in (("fprop", r_fprop), ("dgrad", r_dgrad), ("wgrad", r_wgrad),
                                 ("fprop_nhwc", r_fprop_nhwc)):
                    t_ms = timed(fn, 20, 3, graph_cycle=0 if args.no_graph else len(sets), all_ranks=False) / 20
                    ref_gpu[f"{name}_f32_{hw}x{hw}x{C}"] = round(t_ms * 1e3, 2)
                del sets
                torch.cuda.empty_cache()

    # ---- end to end: the nn.Module on host buffers ------------------------------------
    mods, host = [], []
    for hw, C in STAGES:
        m = o1d.DepthwiseOrientedConv1d(C, C, K, groups=C, padding=K // 2, nhwc=True,
                                        angle=[float(a) for a in round_robin_angles(C)]).to(dev)
        mods.append(m)
        hx = torch.randn((BATCH, hw, hw, C), generator=g).pin_memory()
        hdy = torch.randn((BATCH, hw, hw, C), generator=g).pin_memory()
        hy, hdx = torch.empty_like(hx).pin_memory(), torch.empty_like(hx).pin_memory()
        hdw = torch.empty((C, 1, 1, K)).pin_memory()
        hdb = torch.empty((C,)).pin_memory()
        host.append((hx, hdy, hy, hdx, hdw, hdb))
    h2d = sum(t[0].numel() * 4 + t[1].numel() * 4 for t in host)
    d2h = sum(t[2].numel() * 4 + t[3].numel() * 4 + t[4].numel() * 4 + t[5].numel() * 4 for t in host)

    # Three streams: uploads, the module's forward/backward (current stream), downloads.  PCIe is
    # full duplex, so uploads overlap the downloads of earlier layers and of the previous step
    # (a serving or training loop streams its batches the same way); every byte still crosses
    # the bus inside the timed region, which ends only when the last download has landed.
    s_up, s_down = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

    def e2e_step():
        cur = torch.cuda.current_stream()
        for m, (hx, hdy, hy, hdx, hdw, hdb) in zip(mods, host):
            m.weight.grad = None
            m.bias.grad = None
            with torch.cuda.stream(s_up):
                x = hx.to(dev, non_blocking=True)
                dy = hdy.to(dev, non_blocking=True)
            cur.wait_stream(s_up)
            x.record_stream(cur)
            dy.record_stream(cur)
            x.requires_grad_(True)
            y = m(x)
            y.backward(dy)
            s_down.wait_stream(cur)
            with torch.cuda.stream(s_down):
                for src, dst in ((y.detach(), hy), (x.grad, hdx), (m.weight.grad, hdw), (m.bias.grad, hdb)):
                    src.record_stream(s_down)
                    dst.copy_(src, non_blocking=True)

    e2e_steps = max(4, min(args.steps, 8))

    def e2e_run():
        for _ in range(e2e_steps):
            e2e_step()
        torch.cuda.current_stream().wait_stream(s_down)      # the timed region includes the last download

    e2e_ms = timed(e2e_run, 1, 1)
    e2e_value = BATCH * world * e2e_steps / (e2e_ms / 1e3)

    # ---- CPU baseline (rank 0, bounded sample) ----------------------------------------
    cpu = None
    if rank == 0 and not args.no_cpu:
        loops, kind = cpu_loops()
        threads = host_threads()
        n_img = 16 * threads
        nt = torch.get_num_threads()
        torch.set_num_threads(1)                      # the batch slices are the parallelism
        cpu_step(loops, threads, threads=threads)
        t = cpu_step(loops, n_img, threads=threads)
        torch.set_num_threads(nt)
        cpu = {"value": n_img / t, "unit": "img/s", "cores": threads, "kind": kind,
               "sample": f"{n_img} images at each of the 4 stage shapes (fprop+dgrad+wgrad), fp32 NCHW, {t:.1f} s: "
                         f"the reference's single-threaded loops on {threads} batch slices in {threads} threads"}
    cpu_conv = None
    if rank == 0 and not args.no_cpu:
        try:
            cpu_conv = cpu_conv2d_baseline()
        except Exception as e:              # a reported baseline must not take the line down
            cpu_conv = {"unavailable": repr(e)}

    # ---- the metric's model figure: ConvNeXt-T-1D inference on the same GPUs ------------------
    model_fig = None
    if not args.no_model:
        torch.cuda.empty_cache()
        model_fig = measure_model(10, 3, 256, world, rank, dev, graph=not args.no_graph)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "img/s", "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "stage-sweep: (56,96),(28,192),(14,384),(7,768) x batch 128 per GPU, K=31, "
                                   "stride 1, NHWC, 8 orientations round-robin; fprop+dgrad+wgrad per shape",
                       "l2": "inputs rotate over sets totalling >4x L2, so every launch reads from HBM",
                       "launch": ("eager" if args.no_graph else "CUDA graph of one full input rotation, replayed" if world == 1
                                  else "one CUDA graph per step (kernels only); the NCCL all-reduce of step i runs on "
                                       "its own stream under the kernels of step i+1"),
                       "parallelism": f"dp{world} (batch-sharded; weight-gradient all-reduce when >1)"},
            "roofline": roof, "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": "img/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": n_launch, "clocks": clocks, "kernels": kernels, "kernels_block": kernels_block,
            "reference_gpu_us": ref_gpu, "cpu_conv2d": cpu_conv, "model": model_fig,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_case(args):
    """One kernel on its own, a few launches: the command profiled with ncu.  Case names are
    <op>_<f32|bf16>_<H>x<W>x<C>: the keys of the `kernels` table (fprop, dgrad, wgrad; stride 1,
    K = 31), plus fprop2 / dgrad2 / wgrad2 (stride 2, H x W is the input size), ln (channels-last
    LayerNorm), pw (stem projection from a 3-channel image to C channels) and tr (NHWC -> NCHW
    transpose)."""
    import torch

    import oriented1d_b200 as o1d

    op, tag, shape = args.case.split("_")
    H, W, C = (int(v) for v in shape.split("x"))
    dtype = torch.float32 if tag == "f32" else torch.bfloat16
    es = 4 if dtype == torch.float32 else 2
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device="cpu").manual_seed(0)
    n = args.batch
    stride = 2 if op.endswith("2") else 1
    P, Q = -(-H // stride), -(-W // stride)
    if op == "pw":
        sets = [(torch.randn((n, 3, H, W), generator=g).to(dev).to(dtype), None) for _ in range(2)]
        w = torch.randn((C, 3), generator=g).to(dev)
        bias = torch.randn((C,), generator=g).to(dev)
        alg = n * H * W * (3 + C) * es
    else:
        plan = o1d.Plan(round_robin_angles(C) if args.angles == "rr" else [0.0] * C if args.angles == "zero" else block_angles(C), K)
        w = (0.02 * torch.randn((C, 1, 1, K), generator=g)).to(dev)
        bias = torch.randn((C,), generator=g).to(dev)
        sets = [(torch.randn((n, H, W, C), generator=g).to(dev).to(dtype),
                 torch.randn((n, P, Q, C), generator=g).to(dev).to(dtype)) for _ in range(2)]
        alg = ((n * H * W * C + n * P * Q * C) * es if op not in ("ln", "tr", "lnbwd", "colsum") else
               3 * n * H * W * C * es if op == "lnbwd" else n * H * W * C * es if op == "colsum" else 2 * n * H * W * C * es)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for i in range(args.reps):
        x, dy = sets[i % 2]
        e0.record()
        if op in ("fprop", "fprop2"):
            o1d.fprop(x, w, None, plan, stride, True)
        elif op in ("dgrad", "dgrad2"):
            o1d.dgrad(dy, w, plan, H, W, stride, True)
        elif op in ("wgrad", "wgrad2"):
            o1d.wgrad(dy, x, plan, stride, True, True)
        elif op == "ln":
            o1d.ops.layer_norm_cl(x, bias, bias, 1e-6, False)
        elif op == "lnbwd":
            o1d.ops.layer_norm_cl_bwd(x, dy, bias, 1e-6)
        elif op == "colsum":
            o1d.ops.colsum(dy)
        elif op == "pw":
            o1d.ops.pointwise_in(x, w, bias)
        elif op == "tr":
            o1d.ops.nhwc_to_nchw(x)
        else:
            raise SystemExit("unknown case " + args.case)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3)
    print(json.dumps({"case": args.case, "batch": n, "us": times, "alg_bytes": alg,
                      "device_status": o1d.ops.device_status()}))


def init_ranks():
    """(world, rank, local, device); starts the NCCL process group when launched by torchrun."""
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("NCCL_DEBUG", "WARN")     # keep stdout to the one JSON line
        dist.init_process_group("nccl", device_id=dev)
    return world, rank, local, dev


def timed_steps(fn, steps, warmup, world, dev, graph_cycle=0, tail=None):
    """Device milliseconds of `steps` calls of fn: CUDA events on the launching stream, barrier and
    synchronize on both sides, max over ranks.  graph_cycle > 0 captures that many consecutive
    calls into one CUDA graph and replays it.  `tail` runs after the last call, inside the timed
    region."""
    import torch
    import torch.distributed as dist
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    runner, per = fn, 1
    if graph_cycle > 0:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(graph_cycle):
                fn()
        g.replay()
        runner, per = g.replay, graph_cycle
    reps = max(1, -(-steps // per))
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        runner()
    if tail is not None:
        tail()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = e0.elapsed_time(e1) * steps / (reps * per)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def measure_model(steps, warmup, batch, world, rank, dev, graph=True):
    """ConvNeXt-T-1D full-model inference: depths 3/3/9/3, dims 96..768, K=31 oriented convs in every
    block and in the stem, 1000 classes, random init, bf16, `batch` synthetic N(0,1) 224x224 images per
    GPU, batch-sharded over the GPUs with no collective.  Returns device-resident and end-to-end
    throughput (every batch uploaded from pinned host memory, logits downloaded)."""
    import torch
    import torch.distributed as dist

    from oriented1d_b200 import convnext1d

    torch.manual_seed(rank)
    model = convnext1d.convnext_tiny(variant="1d", drop_path_rate=0.0).to(dev).bfloat16().eval()
    nsets = 3
    imgs = [torch.randn((batch, 3, 224, 224), device=dev).bfloat16() for _ in range(nsets)]
    host_img = torch.randn((batch, 3, 224, 224)).bfloat16().pin_memory()
    host_out = torch.empty((batch, 1000), dtype=torch.bfloat16).pin_memory()
    state = {"i": 0}

    def step():
        state["i"] = (state["i"] + 1) % nsets
        with torch.no_grad():
            return model(imgs[state["i"]])

    # End to end: every batch comes from pinned host memory and the logits go back to it.  Uploads,
    # the forward pass and downloads run on three streams with two device input buffers, so the
    # upload of batch i+1 overlaps the forward pass of batch i (PCIe is full duplex).
    up, down = torch.cuda.Stream(), torch.cuda.Stream()
    dev_in = [torch.empty_like(imgs[0]) for _ in range(2)]
    ev_up = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]
    e2e_state = {"i": 0}

    def e2e_step():
        cur = torch.cuda.current_stream()
        b = e2e_state["i"] & 1
        e2e_state["i"] += 1
        with torch.cuda.stream(up):
            up.wait_event(ev_free[b])                   # the forward pass that last read this buffer
            dev_in[b].copy_(host_img, non_blocking=True)
            ev_up[b].record(up)
        cur.wait_event(ev_up[b])
        with torch.no_grad():
            out = model(dev_in[b])
        ev_free[b].record(cur)
        out.record_stream(down)
        with torch.cuda.stream(down):
            down.wait_event(ev_free[b])
            host_out.copy_(out, non_blocking=True)

    ms = timed_steps(step, steps, max(warmup, 3), world, dev, graph_cycle=nsets if graph else 0)
    n_e2e = max(4, min(steps, 10))
    e2e_ms = timed_steps(e2e_step, n_e2e, 3, world, dev,
                         tail=lambda: torch.cuda.current_stream().wait_stream(down))
    out = {"value": batch * world * steps / (ms / 1e3), "unit": "img/s", "ms_per_step": ms / steps, "batch": batch,
           "e2e": {"value": batch * world * n_e2e / (e2e_ms / 1e3), "unit": "img/s",
                   "h2d_bytes_per_step": host_img.numel() * 2, "d2h_bytes_per_step": host_out.numel() * 2,
                   "ms_per_step": e2e_ms / n_e2e},
           "workload": "ConvNeXt-T-1D inference: depths 3/3/9/3, dims 96-768, K=31, 8 orientations (block-wise per "
                       f"layer), batch {batch} per GPU, 224x224x3 bf16, random init, 1000 classes",
           "gpu_launches_per_step": 20}      # oriented-conv launches per forward: 2 stem convs + 18 block convs
    del model, imgs, dev_in
    torch.cuda.empty_cache()
    return out


def run_model(args):
    import torch.distributed as dist
    world, rank, local, dev = init_ranks()
    batch = args.batch if args.batch != 64 else 256
    with ClockSampler(local) as clk:
        m = measure_model(args.steps, args.warmup, batch, world, rank, dev, graph=not args.no_graph)
        time.sleep(0.25)
    if rank == 0:
        print(json.dumps({
            "metric": "ConvNeXt-T-1D inference throughput @224", "value": m["value"], "unit": "img/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": m["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": m["workload"], "l2": "activations exceed L2; 3 input batches rotate",
                       "launch": "eager" if args.no_graph else "CUDA graph replay",
                       "parallelism": f"dp{world} (batch-sharded, no collective)"},
            "e2e": m["e2e"], "gpu_launches": m["gpu_launches_per_step"] * args.steps, "clocks": clk.summary(),
            "roofline": None, "cpu_baseline": None}))
    if world > 1:
        dist.destroy_process_group()


def flat_gradient_buffer(model):
    """One contiguous fp32/bf16 buffer holding every parameter's gradient (each p.grad is a view into
    it), so that data-parallel training needs one all-reduce per step.  Parameters that never receive
    a gradient (the oriented convs' angles) are left out, which is what spares the reference's
    find_unused_parameters pass (main.py:346-348)."""
    import torch
    params = [p for n, p in model.named_parameters() if p.requires_grad and not n.endswith("theta")]
    total = sum(p.numel() for p in params)
    flat = torch.zeros(total, dtype=params[0].dtype, device=params[0].device)
    off = 0
    for p in params:
        p.grad = flat[off:off + p.numel()].view_as(p)
        off += p.numel()
    return flat, params


def run_train(args):
    """ConvNeXt-B-1D++ data-parallel training step: depths 3/3/27/3, dims 128..1024, blocks with a K=15
    oriented conv and a K=31 one on the 4x hidden tensor, stem K=15; batch 64 per GPU of synthetic
    224x224x3 images with uniform labels in [0,1000), cross-entropy, torch AdamW, one all-reduce of
    the flat gradient buffer (engine.py:29-82, main.py:346-348).  Weights, activations and optimizer
    state in bf16 (no autocast)."""
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    from oriented1d_b200 import convnext1d

    world, rank, local, dev = init_ranks()
    torch.manual_seed(rank)
    batch = args.batch if args.batch != 64 else 64
    model = convnext1d.convnext_base(variant="1dpp", drop_path_rate=0.0, fuse_gelu="auto" if args.fuse_gelu else False)
    model = model.to(dev).bfloat16().train()
    flat, params = flat_gradient_buffer(model)
    opt = torch.optim.AdamW(params, lr=1e-4, weight_decay=0.05, fused=True, capturable=True)
    nsets = 2
    imgs = [torch.randn((batch, 3, 224, 224), device=dev).bfloat16() for _ in range(nsets)]
    labels = [torch.randint(0, 1000, (batch,), device=dev) for _ in range(nsets)]
    host_img = torch.randn((batch, 3, 224, 224)).bfloat16().pin_memory()
    host_lab = torch.randint(0, 1000, (batch,)).pin_memory()
    host_loss = torch.empty((), dtype=torch.float32).pin_memory()
    state = {"i": 0}

    def train_step(x, t):
        flat.zero_()
        loss = F.cross_entropy(model(x).float(), t)
        loss.backward()
        if world > 1:
            dist.all_reduce(flat)
            flat.div_(world)
        opt.step()
        return loss

    # One process, one GPU: the whole step (forward, backward, optimizer) is captured into a CUDA graph
    # after three eager steps and replayed on static input buffers, which takes the ~4000 kernel
    # launches per step off the host.  With several ranks the step stays eager (the all-reduce sits in it).
    static_x, static_t = torch.empty_like(imgs[0]), torch.empty_like(labels[0])
    graph, static_loss, launch = None, None, "eager"
    if not args.no_graph and (world == 1 or args.graph_collective):
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for i in range(3):
                    static_x.copy_(imgs[i % nsets]); static_t.copy_(labels[i % nsets])
                    train_step(static_x, static_t)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_loss = train_step(static_x, static_t)
            launch = "CUDA graph of the whole step" + (" (all-reduce captured)" if world > 1 else "")
        except Exception as e:                      # noqa: BLE001 - any capture failure: run eagerly
            print(f"[bench] step not captured ({type(e).__name__}: {e}); running eagerly", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()

    def run_step(x, t):
        if graph is None:
            return train_step(x, t)
        static_x.copy_(x, non_blocking=True); static_t.copy_(t, non_blocking=True)
        graph.replay()
        return static_loss

    def step():
        state["i"] = (state["i"] + 1) % nsets
        run_step(imgs[state["i"]], labels[state["i"]])

    def e2e_step():
        if graph is None:
            x = host_img.to(dev, non_blocking=True)
            t = host_lab.to(dev, non_blocking=True)
            host_loss.copy_(train_step(x, t).detach(), non_blocking=True)
        else:
            host_loss.copy_(run_step(host_img, host_lab).detach(), non_blocking=True)

    with ClockSampler(local) as clk:
        ms = timed_steps(step, args.steps, max(args.warmup, 3), world, dev)
        time.sleep(0.25)
    n_e2e = max(3, min(args.steps, 6))
    e2e_ms = timed_steps(e2e_step, n_e2e, 2, world, dev)
    n_conv = sum(1 for m in model.modules() if m.__class__.__name__ == "DepthwiseOrientedConv1d")
    if rank == 0:
        print(json.dumps({
            "metric": "ConvNeXt-B-1D++ training throughput @224", "value": batch * world * args.steps / (ms / 1e3),
            "unit": "img/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "ConvNeXt-B-1D++ training step: depths 3/3/27/3, dims 128-1024, K=(15,31), "
                                   f"batch {batch} per GPU, 224x224x3 bf16, cross-entropy, AdamW (fused), random init",
                       "l2": "activations exceed L2; 2 input batches rotate", "launch": launch,
                       "gelu": "inside the second conv's kernels on 56x56 and 28x28 maps" if args.fuse_gelu else "separate pass",
                       "parallelism": f"dp{world}: one NCCL all-reduce of the flat gradient buffer "
                                      f"({flat.numel() * flat.element_size() / 1e6:.0f} MB) per step",
                       "parameters": sum(p.numel() for p in model.parameters())},
            "e2e": {"value": batch * world * n_e2e / (e2e_ms / 1e3), "unit": "img/s",
                    "h2d_bytes_per_step": host_img.numel() * 2 + host_lab.numel() * 8, "d2h_bytes_per_step": 4,
                    "ms_per_step": e2e_ms / n_e2e},
            "gpu_launches": 4 * n_conv * args.steps,      # fprop, dgrad, wgrad (2 kernels) per oriented conv
            "clocks": clk.summary(), "roofline": None, "cpu_baseline": None}), flush=True)
    if world > 1:
        if graph is not None:        # a graph that holds captured collectives goes before the communicator
            torch.cuda.synchronize()
            graph.reset()
            graph = None
        dist.barrier()
        dist.destroy_process_group()


def run_dense(args):
    """Dense-prediction backbone shape: the ConvNeXt-T-1D backbone (kernels cropped to 31/31/27/13, four
    normalised stage outputs; semantic_segmentation/backbone/convnext.py:316-327,433-443), forward +
    backward at 2 x 3 x 800 x 1280 bf16 per GPU, loss = sum of the four outputs' sums; gradients
    all-reduced as one flat buffer when more than one GPU runs."""
    import torch
    import torch.distributed as dist

    from oriented1d_b200 import backbone

    world, rank, local, dev = init_ranks()
    torch.manual_seed(rank)
    batch = args.batch if args.batch != 64 else 2
    model = backbone.backbone_tiny(variant="1d").to(dev).bfloat16().train()
    flat, params = flat_gradient_buffer(model)
    nsets = 2
    imgs = [torch.randn((batch, 3, 800, 1280), device=dev).bfloat16() for _ in range(nsets)]
    host_img = torch.randn((batch, 3, 800, 1280)).bfloat16().pin_memory()
    host_loss = torch.empty((), dtype=torch.float32).pin_memory()
    state = {"i": 0}

    def fwd_bwd(x):
        flat.zero_()
        loss = sum(o.float().sum() for o in model(x))
        loss.backward()
        if world > 1:
            dist.all_reduce(flat)
        return loss

    # one GPU: forward + backward captured into a CUDA graph after three eager passes (see run_train)
    static_x = torch.empty_like(imgs[0])
    graph, static_loss, launch = None, None, "eager"
    if world == 1 and not args.no_graph:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for i in range(3):
                    static_x.copy_(imgs[i % nsets])
                    fwd_bwd(static_x)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_loss = fwd_bwd(static_x)
            launch = "CUDA graph of forward + backward"
        except Exception as e:                      # noqa: BLE001 - any capture failure: run eagerly
            print(f"[bench] pass not captured ({type(e).__name__}: {e}); running eagerly", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()

    def run_pass(x):
        if graph is None:
            return fwd_bwd(x if x.is_cuda else x.to(dev, non_blocking=True))
        static_x.copy_(x, non_blocking=True)
        graph.replay()
        return static_loss

    def step():
        state["i"] = (state["i"] + 1) % nsets
        run_pass(imgs[state["i"]])

    def e2e_step():
        host_loss.copy_(run_pass(host_img).detach(), non_blocking=True)

    with ClockSampler(local) as clk:
        ms = timed_steps(step, args.steps, max(args.warmup, 3), world, dev)
        time.sleep(0.25)
    n_e2e = max(3, min(args.steps, 6))
    e2e_ms = timed_steps(e2e_step, n_e2e, 2, world, dev)
    n_conv = sum(1 for m in model.modules() if m.__class__.__name__ == "DepthwiseOrientedConv1d")
    if rank == 0:
        print(json.dumps({
            "metric": "ConvNeXt-T-1D dense-prediction backbone forward+backward @800x1280",
            "value": batch * world * args.steps / (ms / 1e3), "unit": "img/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"ConvNeXt-T-1D backbone, kernels 31/31/27/13, batch {batch} per GPU, 800x1280x3 bf16, "
                                   "forward + backward, loss = sum of the four stage outputs, random init",
                       "l2": "activations exceed L2", "launch": launch,
                       "parallelism": f"dp{world}: flat gradient all-reduce"},
            "e2e": {"value": batch * world * n_e2e / (e2e_ms / 1e3), "unit": "img/s",
                    "h2d_bytes_per_step": host_img.numel() * 2, "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms / n_e2e},
            "gpu_launches": 4 * n_conv * args.steps, "clocks": clk.summary(), "roofline": None, "cpu_baseline": None}))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-ref-gpu", action="store_true", help="skip timing the reference's CUDA kernels")
    ap.add_argument("--no-graph", action="store_true", help="time eager launches instead of CUDA graphs")
    ap.add_argument("--workload", default="sweep", choices=["sweep", "model", "train", "dense"],
                    help="sweep: kernel sweep at the stage shapes plus the model figure (default); model: "
                         "ConvNeXt-T-1D inference; train: ConvNeXt-B-1D++ training step; dense: backbone at 800x1280")
    ap.add_argument("--case", default=None, help="run one kernel case alone, e.g. fprop_f32_56x56x96")
    ap.add_argument("--batch", type=int, default=64, help="batch for --case")
    ap.add_argument("--reps", type=int, default=3, help="launches for --case")
    ap.add_argument("--angles", default="rr", choices=["rr", "block", "zero"], help="channel->orientation map for --case")
    ap.add_argument("--route", type=int, default=0, choices=[0, 1, 2, 3, 4, 5],
                    help="kernel family: 0 automatic (default), 1 general only, 2 prefer tiled, 3 prefer direct, "
                         "4 prefer whole-line")
    ap.add_argument("--fuse-gelu", action="store_true",
                    help="train workload: apply each block's GELU inside its second oriented conv's kernels")
    ap.add_argument("--graph-collective", action="store_true",
                    help="train workload on several GPUs: capture the step, NCCL all-reduce included, into a CUDA graph")
    ap.add_argument("--no-model", action="store_true", help="sweep workload: skip the model figure")
    args = ap.parse_args()
    if args.route and args.impl == "ours":
        from oriented1d_b200 import ops
        ops.set_route(args.route)
    if args.case:
        run_case(args)
    elif args.workload == "model":
        run_model(args)
    elif args.workload == "train":
        run_train(args)
    elif args.workload == "dense":
        run_dense(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
