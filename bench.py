#!/usr/bin/env python
"""Benchmark of the tensor hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-ops]

One "step" = one pass of eltwise activation forward + backward (relu, tanh, logistic, elu with
alpha = 1) over one fp32 [256,256,28,28] nchw batch: 8 kernel launches through the C ABI,
4 x (411 041 792 + 616 562 688) = 4 110 417 920 algorithmic bytes.  Inputs are synthetic, seeded as
the benchmark configuration states (x normal(0, sigma=2) seed 1, dy normal(0,1) seed 2), resident in
HBM before the timed region, and larger than L2 (205 MB each), so no flush is needed.  With N > 1
(launched under torch.distributed.run) every rank owns one such batch -- weak scaling, no
collective on this path -- and the value is all ranks' bytes over the slowest rank's device time.

Prints ONE JSON line (rank 0): the headline metric, per-kernel roofline of the dominant kernel
(activation backward), an end-to-end figure with host buffers, a CPU baseline from the oracle on a
bounded sample, clocks seen during the timed region, and -- unless --no-ops -- a table of every other
configuration's ops (reorder, broadcast op-tensor, reductions, large reorder + conversion).

`--impl reference` times the CPU restatement of the reference's DNNL path (oracle/, all host
threads) on a bounded sample of the same workload: the reference itself is Clojure on the JVM and
cannot run here.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPE_C2 = [256, 256, 28, 28]
ACTS = [("relu", 0.0), ("tanh", 0.0), ("logistic", 0.0), ("elu", 1.0)]
WORKLOAD = "eltwise activation fwd+bwd (relu,tanh,logistic,elu) fp32 [256,256,28,28] nchw"
METRIC = "HBM GB/s (algorithmic bytes / device time) on the tensor hot path: eltwise activation fwd+bwd"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# ------------------------------------------------------------------ clocks sampler -------------

class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU while the timed region runs: NVML
    (read-only queries) from a thread every few ms, or nvidia-smi in a loop if NVML is missing."""

    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
               "sw_power_cap": 0x4}

    def __init__(self, cuda_index):
        self.cuda_index = cuda_index
        self.sm, self.mx, self.power, self.reasons = [], [], [], set()
        self.stop_flag = threading.Event()
        self.thread = None
        self.how = None

    def _nvml_handle(self):
        import pynvml
        import torch
        pynvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(self.cuda_index).uuid)
        if not uuid.startswith("GPU-"):
            uuid = "GPU-" + uuid
        try:
            return pynvml, pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.cuda_index)

    def _loop_nvml(self, pynvml, hd):
        mx = pynvml.nvmlDeviceGetMaxClockInfo(hd, pynvml.NVML_CLOCK_SM)
        while not self.stop_flag.is_set():
            try:
                self.sm.append(float(pynvml.nvmlDeviceGetClockInfo(hd, pynvml.NVML_CLOCK_SM)))
                self.mx.append(float(mx))
                if len(self.sm) % 16 == 1:
                    self.power.append(pynvml.nvmlDeviceGetPowerUsage(hd) / 1000.0)
                bits = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(hd)
                for name, bit in self.REASONS.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.001)

    def _loop_smi(self):
        q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.cuda_index), "--query-gpu=" + q,
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                r = [c.strip() for c in out.strip().splitlines()[0].split(",")]
                self.sm.append(float(r[0]))
                self.mx.append(float(r[1]))
                self.power.append(float(r[2]))
                for name, v in zip(names, r[3:7]):
                    if v.lower().startswith("active"):
                        self.reasons.add(name)
            except Exception:
                time.sleep(0.05)

    def start(self):
        try:
            pynvml, hd = self._nvml_handle()
            self.how = "nvml"
            self.thread = threading.Thread(target=self._loop_nvml, args=(pynvml, hd), daemon=True)
        except Exception:
            self.how = "nvidia-smi"
            self.thread = threading.Thread(target=self._loop_smi, daemon=True)
        self.thread.start()

    def stop(self):
        self.stop_flag.set()
        if self.thread is not None:
            self.thread.join(timeout=6)
        return {"sm_mhz": float(np.median(self.sm)) if self.sm else None,
                "sm_max_mhz": max(self.mx) if self.mx else None,
                "power_w_max": round(max(self.power), 1) if self.power else None,
                "samples": len(self.sm), "via": self.how, "reasons": sorted(self.reasons)}


# ------------------------------------------------------------------ CPU legs -------------------

def cpu_sample(oracle, n_batch, reps):
    """The eltwise step on a [n_batch,256,28,28] slice with the CPU oracle; returns GB/s."""
    shape = [n_batch] + SHAPE_C2[1:]
    x = oracle.gen_normal(shape, 2.0, 1).reshape(-1)
    dy = oracle.gen_normal(shape, 1.0, 2).reshape(-1)
    y, dx = np.empty_like(x), np.empty_like(x)
    nbytes = x.size * 4 * (2 + 3) * len(ACTS)
    oracle.eltwise_fwd("relu", x, y)  # warm the threads
    t0 = time.perf_counter()
    for _ in range(reps):
        for mode, coef in ACTS:
            oracle.eltwise_fwd(mode, x, y, coef=coef)
            oracle.eltwise_bwd(mode, x, dy, dx, coef=coef)
    dt = (time.perf_counter() - t0) / reps
    return nbytes / dt / 1e9, dt, x.size


def onednn_forward_sample(n_batch=32, reps=3):
    """Real oneDNN (the build inside PyTorch, through mkldnn tensors) on the host cores for what that
    route exposes: the three forward activations, same-shape add / mul and the f32 -> bf16 reorder;
    elements/s and GB/s on a [n_batch,256,28,28] slice.  It has no elu, no backward, no broadcast,
    no reduction and no nhwc reorder, so it complements the oracle's number rather than replacing it."""
    try:
        import torch
        torch.set_num_threads(os.cpu_count() or 1)
        import oracle
        shape = [n_batch] + SHAPE_C2[1:]
        x = torch.from_numpy(oracle.gen_normal(shape, 2.0, 1)).to_mkldnn()
        out = {}
        for name, fn in (("relu", torch.relu), ("logistic", torch.sigmoid), ("tanh", torch.tanh)):
            fn(x)
            t0 = time.perf_counter()
            for _ in range(reps):
                fn(x)
            dt = (time.perf_counter() - t0) / reps
            n = int(np.prod(shape))
            out[name] = {"Gelem/s": round(n / dt / 1e9, 3), "GB/s": round(n * 8 / dt / 1e9, 2)}
        # the other ops this route exposes: same-shape add / mul (binary) and the f32 -> bf16 reorder
        xd = torch.from_numpy(oracle.gen_normal(shape, 2.0, 1))
        y = torch.from_numpy(oracle.gen_normal(shape, 1.0, 2)).to_mkldnn()
        n = int(np.prod(shape))
        for name, fn, nbytes in (("add (same shape)", lambda: torch.add(x, y), n * 12),
                                 ("mul (same shape)", lambda: torch.mul(x, y), n * 12),
                                 ("reorder f32 -> bf16", lambda: xd.to_mkldnn(torch.bfloat16), n * 6)):
            fn()
            t0 = time.perf_counter()
            for _ in range(reps):
                fn()
            dt = (time.perf_counter() - t0) / reps
            out[name] = {"Gelem/s": round(n / dt / 1e9, 3), "GB/s": round(nbytes / dt / 1e9, 2)}
        ver = [ln.strip(" -") for ln in torch.__config__.show().splitlines() if "MKL-DNN" in ln]
        out["library"] = ver[0] if ver else "oneDNN (version unknown)"
        out["threads"] = torch.get_num_threads()
        return out
    except Exception as e:  # mkldnn tensors unavailable: report that, the oracle number stands
        return {"unavailable": str(e)[:200]}


def run_reference(args):
    import oracle
    oracle.build()
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    oracle.set_num_threads(os.cpu_count() or 1)  # all host threads, whatever the launcher exported
    n_batch = 32
    vals = []
    for _ in range(args.warmup):
        cpu_sample(oracle, n_batch, 1)
    t_all = 0.0
    for _ in range(args.steps):
        gbs, dt, _ = cpu_sample(oracle, n_batch, 1)
        vals.append(gbs)
        t_all += dt
    value = float(np.mean(vals))
    sample = "per step: the 8 eltwise ops on a [%d,256,28,28] slice (1/%d of the batch)" % (n_batch, SHAPE_C2[0] // n_batch)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t_all / max(args.steps, 1),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": WORKLOAD, "l2": "inputs larger than L2"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": oracle.num_threads(), "kind": "port",
                         "sample": sample, "onednn_forward_via_torch": onednn_forward_sample()},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference is Clojure on the JVM calling oneDNN; no JVM on this box, so this arm "
                "times oracle/ (the CPU restatement of its DNNL path, OpenMP, all host threads)",
    }
    print(json.dumps(line))


# ------------------------------------------------------------------ GPU helpers ----------------

def event_ms(torch, fn, stream, reps, warm):
    """Per-launch device time with one CUDA-event pair per launch (used where a launch cannot be
    captured in a graph, i.e. the NCCL path).  Includes any host launch gap."""
    for _ in range(warm):
        fn()
    stream.synchronize()
    evs = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        fn()
        b.record(stream)
        evs.append((a, b))
    stream.synchronize()
    t = sorted(a.elapsed_time(b) for a, b in evs)
    return t[len(t) // 2], t[max(0, len(t) // 10)], t[min(len(t) - 1, (9 * len(t)) // 10)]


def graph_ms(torch, fact, fn, per_graph, replays, warm=20):
    """Per-launch device time of `fn` (one library call = one kernel) with the host taken out of the
    loop: `per_graph` calls are captured into a CUDA graph on a side stream, the graph is replayed
    `replays` times with an event pair around each replay, and the median replay time is divided by
    the launches it holds.  A Python + ctypes call costs 10-20 us of host time, more than the
    smaller kernels run, so timing un-captured launches would measure the host."""
    h = fact.handle
    side = torch.cuda.Stream(device=fact.device)
    side.wait_stream(fact.stream)
    h.set_stream(side)
    try:
        with torch.cuda.stream(side):
            for _ in range(warm):
                fn()
            side.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for _ in range(per_graph):
                    fn()
            g.replay()
            side.synchronize()
            evs = []
            for _ in range(replays):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(side)
                g.replay()
                b.record(side)
                evs.append((a, b))
            side.synchronize()
    finally:
        h.set_stream(fact.stream)
    t = sorted(a.elapsed_time(b) / per_graph for a, b in evs)
    return t[len(t) // 2], t[max(0, len(t) // 10)], t[min(len(t) - 1, (9 * len(t)) // 10)]


def op_row(name, cfg, nbytes, ms, peak, elems):
    med, p10, p90 = ms
    gbs = nbytes / (med * 1e-3) / 1e9
    return {"op": name, "config": cfg, "algorithmic_bytes": int(nbytes), "ms": round(med, 5),
            "ms_p10": round(p10, 5), "ms_p90": round(p90, 5), "GB/s": round(gbs, 1),
            "frac_of_measured_peak": round(gbs / peak, 4), "frac_of_nominal_8TBs": round(gbs / NOMINAL_HBM_GBS, 4),
            "Gelem/s": round(elems / (med * 1e-3) / 1e9, 2)}


def ops_table(torch, fact, core, oracle, peak, sharded=None, world=1, profile_only=False, c5_batch=None):
    """Every other configuration's ops, each timed alone: launches captured in a CUDA graph and
    replayed between CUDA events (see graph_ms).  Small tensors rotate through enough distinct
    buffers to exceed L2, so every launch is cold.  With `profile_only` each op is just launched
    three times (a short, fixed launch list for a profiler) and nothing is timed."""
    rows = []
    h, dev, stream = fact.handle, fact.device, fact.stream
    L2 = 126 << 20
    it = [0]

    def dbuf(nbytes):
        return torch.empty(int(nbytes), dtype=torch.uint8, device=dev)

    def put(arr):
        return torch.from_numpy(np.ascontiguousarray(arr).reshape(-1).view(np.uint8)).to(dev)

    def measure(name, cfg, nbytes, elems, fn, per_graph, replays, graph=True):
        if profile_only:
            for _ in range(3):
                fn()
            stream.synchronize()
            rows.append({"op": name, "config": cfg, "kernel": h.last_kernel()})
            return
        if graph:
            ms = graph_ms(torch, fact, fn, per_graph, replays)
        else:
            ms = event_ms(torch, fn, stream, 100, 10)
        row = op_row(name, cfg, nbytes, ms, peak, elems)
        row["kernel"] = h.last_kernel()
        rows.append(row)

    # C1: fp32 [32,64,56,56] nchw -> nhwc (25.7 MB each way: rotate buffer pairs past L2)
    shp = [32, 64, 56, 56]
    n = int(np.prod(shp))
    xd = core.tensor_descriptor(shp, "float", "nchw")
    yd = core.tensor_descriptor(shp, "float", "nhwc")
    x0 = put(oracle.gen_uniform(shp, -1, 1, 0))
    sets = max(2, (2 * L2) // (n * 8) + 1)
    xs = [x0] + [x0.clone() for _ in range(sets - 1)]
    ys = [dbuf(n * 4) for _ in range(sets)]

    def c1():
        i = it[0] % sets
        it[0] += 1
        core.transform_tensor(h, 1.0, xd, xs[i], 0.0, yd, ys[i])

    def c1w():
        core.transform_tensor(h, 1.0, xd, xs[0], 0.0, yd, ys[0])
    measure("reorder f32 nchw->nhwc", "C1 [32,64,56,56], cold L2 (rotating %d buffer pairs)" % sets, n * 8, n, c1, 4 * sets, 20)
    measure("reorder f32 nchw->nhwc (warm L2)", "C1 [32,64,56,56], same buffers every launch", n * 8, n, c1w, 24, 20)
    del xs, ys

    # C3: broadcast op-tensor on [128,512,14,14]
    shp = [128, 512, 14, 14]
    n = int(np.prod(shp))
    xd = core.tensor_descriptor(shp, "float", "nchw")
    bd = core.tensor_descriptor([1, 512, 1, 1], "float", "nchw")
    bias = put(oracle.gen_uniform([512], -0.1, 0.1, 4))
    scale = put(oracle.gen_uniform([512], 0.5, 1.5, 1004))
    x0 = put(oracle.gen_uniform(shp, -1, 1, 3))
    sets = max(2, (2 * L2) // (n * 8) + 1)
    xs = [x0] + [x0.clone() for _ in range(sets - 1)]
    outs = [dbuf(n * 4) for _ in range(sets)]

    def c3add():
        i = it[0] % sets
        it[0] += 1
        core.op_tensor(h, "add", 1.0, xd, xs[i], 0.5, bd, bias, 0.0, xd, outs[i])

    def c3mul():
        i = it[0] % sets
        it[0] += 1
        core.op_tensor(h, "mul", 1.0, xd, xs[i], 1.0, bd, scale, 0.0, xd, outs[i])
    measure("op-tensor a*x + b*bias[c]", "C3 [128,512,14,14], a=1 b=0.5, cold L2", n * 8 + 2048, n, c3add, 4 * sets, 20)
    measure("op-tensor x * scale[c]", "C3 [128,512,14,14], cold L2", n * 8 + 2048, n, c3mul, 4 * sets, 20)
    del xs, outs

    # C4: reductions on [64,1024,32,32] (268 MB: larger than L2).  With world > 1 each rank holds
    # N/world images and the (N,H,W) reductions all-reduce 4 KB.
    full = [64, 1024, 32, 32]
    shp = [full[0] // world] + full[1:]
    n = int(np.prod(shp))
    xd = core.tensor_descriptor(shp, "float", "nchw")
    x = put(oracle.gen_signed_lognormal(shp, 5 + 100 * (sharded.rank if sharded else 0)))
    for op, yshape, label in (("add", [1, 1024, 1, 1], "sum over (N,H,W)"), ("avg", [1, 1024, 1, 1], "mean over (N,H,W)"),
                              ("max", [shp[0], 1, 32, 32], "max over C"), ("norm2", [shp[0], 1, 1, 1], "norm2 over (C,H,W)")):
        yd = core.tensor_descriptor(yshape, "float", "nchw")
        y = dbuf(int(np.prod(yshape)) * 4)
        rtd = core.reduce_tensor_descriptor(op, "float")
        spans = sharded is not None and yshape[0] == 1
        nb = n * 4 + int(np.prod(yshape)) * 4
        if spans:
            fn = lambda rtd=rtd, yd=yd, y=y: sharded.reduce_tensor(rtd, 1.0, xd, x, 0.0, yd, y, spans=True)  # noqa: E731
            if sharded.peer_attached:
                sharded.peer_configure(use_peer=True)
                measure("reduce " + label, "C4 shard [%d,1024,32,32] + 4 KB peer-exchange kernel over NVLink" % shp[0],
                        nb, n, fn, 10, 20)
                if op == "add":
                    sharded.peer_configure(use_peer=True, fused=True)
                    measure("reduce " + label + " (exchange fused into the reduce kernel)",
                            "C4 shard [%d,1024,32,32] + 4 KB pushed over NVLink from inside the reduce kernel" % shp[0],
                            nb, n, fn, 10, 20)
                    sharded.peer_configure(use_peer=True)
                sharded.peer_status()
            if op == "add" or not sharded.peer_attached:
                sharded.peer_configure(use_peer=False)
                measure("reduce " + label + " (NCCL)",
                        "C4 shard [%d,1024,32,32] + 4 KB ncclAllReduce + finish kernel (un-captured launches)" % shp[0],
                        nb, n, fn, 10, 20, graph=False)
                sharded.peer_configure(use_peer=True)
        else:
            fn = lambda rtd=rtd, yd=yd, y=y: core.reduce_tensor(h, rtd, 1.0, xd, x, 0.0, yd, y)  # noqa: E731
            measure("reduce " + label, "C4 [%d,1024,32,32]" % shp[0], nb, n, fn, 10, 20)
    del x

    # C5: [2048/world,256,28,28] f32 nchw -> bf16 nhwc, then s8 nchw -> s8 nhwc
    full = [2048, 256, 28, 28]
    shp = [c5_batch or full[0] // world] + full[1:]
    n = int(np.prod(shp))
    xd = core.tensor_descriptor(shp, "float", "nchw")
    yd = core.tensor_descriptor(shp, "bf16", "nhwc")
    qd = core.tensor_descriptor(shp, "byte", "nchw")
    zd = core.tensor_descriptor(shp, "byte", "nhwc")
    g = torch.Generator(device=dev)
    g.manual_seed(6)
    x = torch.randn(n, dtype=torch.float32, device=dev, generator=g)  # values only feed the timing
    y = dbuf(n * 2)
    q = torch.clamp(torch.round(x * 127.0), -128, 127).to(torch.int8)
    z = dbuf(n)
    measure("reorder+convert f32 nchw -> bf16 nhwc", "C5 [%d,256,28,28]" % shp[0], n * 6, n,
            lambda: core.transform_tensor(h, 1.0, xd, x, 0.0, yd, y), 5, 10)
    measure("reorder s8 nchw -> nhwc", "C5 [%d,256,28,28]" % shp[0], n * 2, n,
            lambda: core.transform_tensor(h, 1.0, qd, q, 0.0, zd, z), 5, 10)
    return rows


class _View:
    """A (descriptor, device address) pair for the entry points that take tensor-like arguments."""

    def __init__(self, desc, buf, byte_offset=0):
        self.desc, self.buf, self.off = desc, buf, int(byte_offset)

    def device_ptr(self):
        return self.buf.data_ptr() + self.off


def next_rows_table(torch, fact, core, oracle, peak, profile_only=False):
    """The callers either side of the path, each timed alone like the per-op table: shuffler gather,
    branch / concatenate copies, n-ary sum, cost, equality, same-layout convert, fill and scale.
    Every tensor is [256,256,28,28]-sized (205 MB in f32) or larger than L2 in total, so launches
    stream from HBM."""
    rows = []
    h, dev, stream = fact.handle, fact.device, fact.stream

    def dbuf(nbytes):
        return torch.empty(int(nbytes), dtype=torch.uint8, device=dev)

    def measure(name, cfg, nbytes, elems, fn, per_graph=5, replays=10):
        if profile_only:
            for _ in range(3):
                fn()
            stream.synchronize()
            rows.append({"op": name, "config": cfg, "kernel": h.last_kernel()})
            return
        row = op_row(name, cfg, nbytes, graph_ms(torch, fact, fn, per_graph, replays), peak, elems)
        row["kernel"] = h.last_kernel()
        rows.append(row)

    g = torch.Generator(device=dev)
    g.manual_seed(7)
    shp = [256, 256, 28, 28]
    n = int(np.prod(shp))
    x = torch.randn(n, dtype=torch.float32, device=dev, generator=g)
    y = torch.empty(n, dtype=torch.float32, device=dev)
    z = torch.randn(n, dtype=torch.float32, device=dev, generator=g)
    d4 = core.tensor_descriptor(shp, "float", "nchw")

    # same-layout convert f32 -> bf16 (flat stream)
    yb = dbuf(n * 2)
    measure("convert f32 -> bf16, same layout", "[256,256,28,28] nchw", n * 6, n,
            lambda: core.transform_tensor(h, 1.0, d4, x, 0.0, core.tensor_descriptor(shp, "bf16", "nchw"), yb))

    # a channel window of a wider tensor copied out (what view-tz + transformer do): rows kernel
    wide = torch.randn(256 * 320 * 784, dtype=torch.float32, device=dev, generator=g)
    wd = core.tensor_descriptor(shp, "float", [320 * 784, 784, 28, 1])
    measure("sub-tensor copy (256 of 320 channels)", "[256,256,28,28] f32 window of [256,320,28,28]", n * 8, n,
            lambda: core.transform_tensor(h, 1.0, wd, wide, 0.0, d4, y))
    del wide
    # relu forward on the same kind of window, into a dense tensor
    ad = core.activation_descriptor("relu", True, 0.0)
    wide = torch.randn(256 * 320 * 784, dtype=torch.float32, device=dev, generator=g)
    measure("relu forward on a sub-tensor view", "[256,256,28,28] f32 window of [256,320,28,28] -> dense", n * 8, n,
            lambda: core.activation_forward(h, ad, 1.0, wd, wide, 0.0, d4, y))
    del wide
    # activations on 16-bit tensors (arithmetic in float): relu and tanh forward on bf16
    db = core.tensor_descriptor(shp, "bf16", "nchw")
    xb = (x.view(torch.int32) >> 16).to(torch.int16)          # the bf16 bit patterns of x (truncated)
    yb16 = dbuf(n * 2)
    for mode in ("relu", "tanh"):
        adm = core.activation_descriptor(mode, True, 0.0)
        measure("%s forward, bf16 tensors" % mode, "[256,256,28,28] bf16", n * 4, n,
                lambda adm=adm: core.activation_forward(h, adm, 1.0, db, xb, 0.0, db, yb16))
    del xb, yb16
    # N and C swapped (nchw -> cnhw): rows of 784 elements
    measure("reorder nchw -> cnhw", "[256,256,28,28] f32", n * 8, n,
            lambda: core.transform_tensor(h, 1.0, d4, x, 0.0,
                                          core.tensor_descriptor(shp, "float", [784, 256 * 784, 28, 1]), y))

    # shuffler: 8192 of 16384 rows of [16384,64,8,8] f32 picked at random into [8192,64,8,8]
    rows_src, rows_dst, row_elems = 16384, 8192, 64 * 8 * 8
    src = torch.randn(rows_src * row_elems, dtype=torch.float32, device=dev, generator=g)
    dst = torch.empty(rows_dst * row_elems, dtype=torch.float32, device=dev)
    perm = np.random.default_rng(8).permutation(rows_src)[:rows_dst]
    sub = core.tensor_descriptor([1, 64, 8, 8], "float", "nchw")
    so, do = [int(i) * row_elems for i in perm], [i * row_elems for i in range(rows_dst)]

    def shuffle():
        for k in range(0, rows_dst, 4096):      # the entry point takes up to 4096 items per call
            core.gather_transform(h, so[k:k + 4096], do[k:k + 4096], sub, src, sub, dst)
    measure("shuffler gather", "8192 random rows of [16384,64,8,8] f32 (16 KB each), 2 calls", rows_dst * row_elems * 8,
            rows_dst * row_elems, shuffle, 2, 10)
    del src, dst

    # branch: [256,256,28,28] cut 64/128/64 along channels, one launch; concatenate is the inverse
    parts, pairs, c0 = [64, 128, 64], [], 0
    outs = []
    for c in parts:
        pshape = [256, c, 28, 28]
        pd_src = core.tensor_descriptor(pshape, "float", [256 * 784, 784, 28, 1])   # a channel window of x
        pd_dst = core.tensor_descriptor(pshape, "float", "nchw")
        o = torch.empty(int(np.prod(pshape)), dtype=torch.float32, device=dev)
        outs.append((pd_dst, o))
        pairs.append((_View(pd_src, x, c0 * 784 * 4), _View(pd_dst, o)))
        c0 += c
    measure("branch (3 sub-tensor copies, one launch)", "[256,256,28,28] f32 -> 64/128/64 channels", n * 8, n,
            lambda: core.multi_transform(h, pairs))
    back = [(b, a) for a, b in pairs]
    measure("concatenate (3 sub-tensor copies, one launch)", "64/128/64 channels -> [256,256,28,28] f32", n * 8, n,
            lambda: core.multi_transform(h, back))
    del outs, pairs, back

    # n-ary sum: y = x + 0.5*z + 0.25*y0 in one pass (3 sources)
    w = torch.randn(n, dtype=torch.float32, device=dev, generator=g)
    measure("sum of 3 tensors, one pass", "[256,256,28,28] f32, scales 1, 0.5, 0.25", n * 16, n,
            lambda: core.sum_tensors(h, [1.0, 0.5, 0.25], [d4, d4, d4], [x, z, w], d4, y))
    del w

    # cost: d = a - y with the quadratic cost / the cross-entropy in the same pass
    cost = torch.zeros(1, dtype=torch.float64, device=dev)
    a01 = torch.rand(n, dtype=torch.float32, device=dev, generator=g) * 0.98 + 0.01
    t01 = (torch.rand(n, dtype=torch.float32, device=dev, generator=g) < 0.1).to(torch.float32)
    d2 = core.tensor_descriptor([256, 256 * 784], "float", "nc")
    measure("cost: a - y and quadratic cost, one pass", "[256, 200704] f32", n * 12, n,
            lambda: core.cost_diff(h, "quadratic", d2, a01, t01, y, cost))
    measure("cost: cross-entropy (no gradient written)", "[256, 200704] f32", n * 8, n,
            lambda: core.cost_diff(h, "crossentropy", d2, a01, t01, None, cost))
    del a01, t01

    # equality of two tensors
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    y.copy_(x)
    measure("tensor equality", "[256,256,28,28] f32 vs an equal copy", n * 8, n,
            lambda: core.tensor_equals(h, d4, x, d4, y, flag))

    # fill and scale
    measure("set-tensor (fill)", "[256,256,28,28] f32", n * 4, n, lambda: core.set_tensor(h, d4, y, 0.5))
    measure("scale-tensor", "[256,256,28,28] f32", n * 8, n, lambda: core.scale_tensor(h, 1.0009765625, d4, y))
    return rows


def run_profile_ops(args):
    """`--profile-ops`: launches every op of the per-op table three times on cuda:0 and prints the
    kernel family each call chose.  A short fixed launch list for ncu; the large reorder runs on a
    per-GPU shard ([256,256,28,28], what one of 8 GPUs holds) to keep the capture small."""
    import torch
    import oracle
    from deep_diamond_b200 import b200_factory, core
    torch.cuda.set_device(0)
    oracle.build()
    fact = b200_factory(0)
    if args.profile_next:
        rows = next_rows_table(torch, fact, core, oracle, peaks()[0], profile_only=True)
    else:
        rows = ops_table(torch, fact, core, oracle, peaks()[0], None, 1, profile_only=True, c5_batch=256)
    print(json.dumps({"profile_ops": rows}))
    fact.release()


# ------------------------------------------------------------------ main GPU arm ---------------

def run_ours(args):
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")  # keep stdout to the one JSON line
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    import oracle
    from deep_diamond_b200 import b200_factory, core, dnn, sharded as shd, tensor as T
    if rank == 0:
        oracle.build()
    fact = b200_factory(local_rank)
    h, stream = fact.handle, fact.stream
    peak, peak_kind = peaks()

    n = int(np.prod(SHAPE_C2))
    x_host = oracle.gen_normal(SHAPE_C2, 2.0, 1 + 1000 * rank).reshape(-1)
    dy_host = oracle.gen_normal(SHAPE_C2, 1.0, 2 + 1000 * rank).reshape(-1)
    d = core.tensor_descriptor(SHAPE_C2, "float", "nchw")
    x = torch.from_numpy(x_host).to(fact.device)
    dy = torch.from_numpy(dy_host).to(fact.device)
    y = torch.empty_like(x)
    dx = torch.empty_like(x)
    ads = [(m, core.activation_descriptor(m, True, c)) for m, c in ACTS]
    fwd_bytes, bwd_bytes = n * 8, n * 12
    step_bytes = len(ACTS) * (fwd_bytes + bwd_bytes)

    def step(events=None):
        for m, ad in ads:
            if events is not None:
                e0 = torch.cuda.Event(enable_timing=True)
                e0.record(stream)
            core.activation_forward(h, ad, 1.0, d, x, 0.0, d, y)
            if events is not None:
                e1 = torch.cuda.Event(enable_timing=True)
                e1.record(stream)
            core.activation_backward(h, ad, 1.0, d, y, d, dy, d, x, 0.0, d, dx)
            if events is not None:
                e2 = torch.cuda.Event(enable_timing=True)
                e2.record(stream)
                events.append((m, e0, e1, e2))

    for _ in range(max(args.warmup, 3)):
        step()
    stream.synchronize()
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # keep the sampled window long enough for nvidia-smi to see it under load
    launches0 = h.launch_count()
    events = []
    t_start, t_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t_start.record(stream)
    for _ in range(args.steps):
        step(events)
    t_stop.record(stream)
    stream.synchronize()
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    launches = h.launch_count() - launches0
    total_ms = t_start.elapsed_time(t_stop)
    if dist:
        t = torch.tensor([total_ms], dtype=torch.float64, device=fact.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    # the timed region lasts milliseconds, one or two NVML samples: keep the same step running for
    # another 0.3 s (untimed) so that the clock record under this load is more than that
    n_timed = len(sampler.sm)
    t_end = time.perf_counter() + 0.3
    while time.perf_counter() < t_end:
        for _ in range(8):
            step()
        stream.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["samples_in_timed_region"] = n_timed
        clocks["sm_mhz_in_timed_region"] = float(np.median(sampler.sm[:n_timed])) if n_timed else None
        clocks["window"] = "timed steps + 0.3 s of the same step"

    fwd_ms = {m: [] for m, _ in ACTS}
    bwd_ms = {m: [] for m, _ in ACTS}
    for m, e0, e1, e2 in events:
        fwd_ms[m].append(e0.elapsed_time(e1))
        bwd_ms[m].append(e1.elapsed_time(e2))
    value = world * args.steps * step_bytes / (total_ms * 1e-3) / 1e9
    all_bwd = [v for m in bwd_ms for v in bwd_ms[m]]
    bwd_avg_ms = float(np.mean(all_bwd))
    achieved = bwd_bytes / (bwd_avg_ms * 1e-3) / 1e9
    per_kernel = {}
    for m, _ in ACTS:
        per_kernel[m] = {
            "fwd_ms": round(float(np.mean(fwd_ms[m])), 5), "fwd_GB/s": round(fwd_bytes / np.mean(fwd_ms[m]) / 1e6, 1),
            "bwd_ms": round(float(np.mean(bwd_ms[m])), 5), "bwd_GB/s": round(bwd_bytes / np.mean(bwd_ms[m]) / 1e6, 1)}

    # parity spot check of what was just timed (last activation = elu): a slice against the oracle
    parity = None
    if rank == 0:
        k = 1 << 16
        got_y = y[:k].cpu().numpy()
        got_dx = dx[:k].cpu().numpy()
        want_y = oracle.eltwise_fwd("elu", x_host[:k], np.empty(k, np.float32), coef=1.0)
        want_dx = oracle.eltwise_bwd("elu", x_host[:k], dy_host[:k], np.empty(k, np.float32), coef=1.0)
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        from conftest import ulp_diff_f32
        parity = {"elu_fwd_max_ulp": int(ulp_diff_f32(got_y, want_y).max()),
                  "elu_bwd_max_ulp": int(ulp_diff_f32(got_dx, want_dx).max()), "checked_elements": k}

    # end to end through the public API with pinned HOST buffers: upload x and dy, run the 8 ops as
    # layers, read y and dx of the last activation back
    tz_x = T.tensor(fact, SHAPE_C2, "float", "nchw")
    tz_dx = T.tensor(fact, SHAPE_C2, "float", "nchw")
    pin_x = torch.from_numpy(x_host).pin_memory()
    pin_dy = torch.from_numpy(dy_host).pin_memory()
    pin_y = torch.empty(n, dtype=torch.float32).pin_memory()
    pin_dx = torch.empty(n, dtype=torch.float32).pin_memory()
    layers = [dnn.activation(fact, tz_x, m, {"alpha": c})(tz_x, tz_dx) for m, c in ACTS]

    # Uploads and downloads go through transfer_async: each direction has its own copy stream, so
    # the download of a result overlaps the next upload (PCIe is full duplex).  y is read back from
    # the logistic layer, the one whose output is not also the buffer its gradient arrives in.
    logistic = [l for l, (m, _) in zip(layers, ACTS) if m == "logistic"][0]
    pend = {"y": None, "dx": None}

    def e2e_step():
        T.transfer_async(pin_x.numpy(), tz_x)
        for layer in layers:
            if layer is logistic and pend["y"] is not None:
                pend["y"].before_overwrite()          # last step's y is still being read from this buffer
            layer.forward()
            if layer is logistic:
                pend["y"] = T.transfer_async(layer.output(), pin_y.numpy())
            # the upstream gradient arrives in the layer's diff-input buffer (which, as in the
            # reference, is the output buffer for every activation but logistic)
            T.transfer_async(pin_dy.numpy(), layer.diff_input())
            if layer is layers[0] and pend["dx"] is not None:
                pend["dx"].before_overwrite()         # every backward writes the shared dx
            layer.backward()
        pend["dx"] = T.transfer_async(tz_dx, pin_dx.numpy())

    def e2e_drain():
        for p in pend.values():
            if p is not None:
                p.wait()

    e2e_steps = 0 if args.no_e2e else max(1, min(args.steps, 10))
    if e2e_steps:
        e2e_step()
        e2e_drain()
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_drain()
    torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - t0) / max(e2e_steps, 1)
    if dist:
        t = torch.tensor([e2e_s], dtype=torch.float64, device=fact.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e = None if args.no_e2e else {"value": round(world * step_bytes / e2e_s / 1e9, 2), "unit": "GB/s",
           "h2d_bytes_per_step": n * 4 * (1 + len(ACTS)), "d2h_bytes_per_step": n * 8,
           "ms_per_step": round(e2e_s * 1e3, 3),
           "api": "tensor.transfer_async (pinned numpy <-> device, uploads and downloads on separate copy streams), "
                  "dnn.activation layers forward/backward"}
    if e2e is not None and rank == 0:
        # what came back over the pipelined copies: y = logistic(x), dx = elu'(x) * dy (the last layer)
        k = 1 << 16
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        from conftest import ulp_diff_f32
        wy = oracle.eltwise_fwd("logistic", x_host[:k], np.empty(k, np.float32))
        wdx = oracle.eltwise_bwd(ACTS[-1][0], x_host[:k], dy_host[:k], np.empty(k, np.float32), coef=ACTS[-1][1])
        e2e["result_max_ulp"] = {"y": int(ulp_diff_f32(pin_y.numpy()[:k], wy).max()),
                                 "dx": int(ulp_diff_f32(pin_dx.numpy()[:k], wdx).max())}
    del layers, tz_x, tz_dx, pin_x, pin_dy, pin_y, pin_dx

    ops = ops_next = None
    if not args.no_ops:
        sh = shd.create_from_torch_distributed(fact) if world > 1 else None
        del x, dy, y, dx
        torch.cuda.empty_cache()
        ops = ops_table(torch, fact, core, oracle, peak, sh, world)
        if sh is not None:
            sh.release()
        torch.cuda.empty_cache()
        ops_next = next_rows_table(torch, fact, core, oracle, peak) if world == 1 else None

    cpu = None
    if rank == 0 and world == 1:
        oracle.set_num_threads(os.cpu_count() or 1)
        gbs, dt, elems = cpu_sample(oracle, 32, 3)
        cpu = {"value": round(gbs, 3), "unit": "GB/s", "cores": oracle.num_threads(), "kind": "port",
               "Gelem/s": round(elems * len(ACTS) * 2 / dt / 1e9, 4),
               "sample": "the 8 eltwise ops on a [32,256,28,28] slice (1/8 of the batch), 3 repetitions, oracle/ (C + OpenMP)",
               "onednn_forward_via_torch": onednn_forward_sample()}

    if rank == 0:
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(total_ms / args.steps, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "bytes_per_step_per_gpu": step_bytes,
                       "l2": "inputs larger than L2 (205 MB per tensor vs 126 MB), no flush needed",
                       "parallelism": "one process per GPU, batch-sharded, no collective on this path"},
            "frac_of_measured_peak": round(value / world / peak, 4),
            "roofline": {"bound": "hbm", "kernel": "dd_elt_flat_kernel<float,float,MODE,BWD=true> (activation backward)",
                         "achieved": round(achieved, 1), "peak": peak, "peak_kind": "of " + peak_kind, "unit": "GB/s",
                         "frac": round(achieved / peak, 4), "frac_of_nominal_8TBs": round(achieved / NOMINAL_HBM_GBS, 4),
                         # dram__bytes_read.sum + dram__bytes_write.sum per backward launch, mean of the four
                         # activations in profiles/eltwise_flat_kernel_ncu_full.md (reads 411.1 MB = the
                         # algorithmic input; writes 173.8 MB: the tail of dx is still in L2 at kernel end)
                         "traffic": 584.8e6, "traffic_source": "ncu capture, profiles/eltwise_flat_kernel_ncu_full.md",
                         "avg_launch_ms": round(bwd_avg_ms, 5),
                         "algorithmic_bytes_per_launch": bwd_bytes},
            "per_kernel": per_kernel,
            "cpu_baseline": cpu,
            "e2e": e2e,
            "gpu_launches": int(launches),
            "clocks": clocks,
            "parity_spot_check": parity,
            "ops": ops,
            "ops_next": ops_next,
        }
        print(json.dumps(line))
    fact.release()
    if dist:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-ops", action="store_true", help="skip the per-op table of the other configurations")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg (for profiler captures)")
    ap.add_argument("--profile-next", action="store_true",
                    help="like --profile-ops for the table of the path's callers (shuffler, branch, sum, cost ...)")
    ap.add_argument("--profile-ops", action="store_true",
                    help="launch each op of the per-op table three times and exit (for profiler captures)")
    args = ap.parse_args()
    if args.profile_ops or args.profile_next:
        run_profile_ops(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
