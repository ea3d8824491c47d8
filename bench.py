#!/usr/bin/env python
"""Benchmark of the tensor hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-ops]

One "pass" = eltwise activation forward + backward (relu, tanh, logistic, elu with alpha = 1) over
one fp32 [256,256,28,28] nchw batch: 8 kernel launches through the C ABI,
4 x (411 041 792 + 616 562 688) = 4 110 417 920 algorithmic bytes.  One "step" = PASSES_PER_STEP
such passes back to back, so that the K timed steps last about half a second and clock samples fall
inside the timed region; the value is all bytes over the whole region (the sustained rate), the
best single pass is reported beside it as the burst rate.  Inputs are synthetic, seeded as the
benchmark configuration states (x normal(0, sigma=2) seed 1, dy normal(0,1) seed 2), resident in
HBM before the timed region, and larger than L2 (205 MB each), so no flush is needed.  With N > 1
(launched under torch.distributed.run) every rank owns one such batch -- weak scaling, no
collective on this path -- and the value is all ranks' bytes over the slowest rank's device time.

Prints ONE JSON line (rank 0): the headline metric, per-kernel roofline of the dominant kernel
(activation backward), an end-to-end figure with host buffers, a CPU baseline (oracle port and real
oneDNN where torch exposes it), clocks seen during the timed region, and -- unless --no-ops -- a
table of every other configuration's ops (reorder, broadcast op-tensor, reductions, large reorder +
conversion).  With N > 1 the reductions that span the sharded batch are first CHECKED against the
oracle's reduction of the whole tensor on every combine path, and the line ends with a compact
`scaling_summary` (per sharded op: time on one GPU for the whole tensor, time per rank, speed-up).

`--impl reference` times the reference's CPU path for the same pass on the full batch with all host
threads: real oneDNN (the build inside PyTorch, through mkldnn tensors) for the three forward
activations it exposes, the CPU restatement in oracle/ for elu and the four backward passes.  The
reference itself is Clojure on the JVM and cannot run here.
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
# dram__bytes_read.sum + dram__bytes_write.sum of ONE activation-backward launch on the bench's
# [256,256,28,28] tensors, from the ncu capture named here (refresh it when the activation kernels change)
TRAFFIC_BWD = {"bytes": 578.6e6, "profile": "profiles/eltwise_backward_dram_traffic.md",
               "captured_at_commit": "7b2758d", "captured_on": "2026-11-25",
               "note": "reads 411.1 MB = the algorithmic input; writes 167.5 MB (the tail of dx is still in L2 when the "
                       "kernel ends) against 616.6 MB algorithmic"}
PASSES_PER_STEP = 36          # 36 passes x 0.71 ms: 20 steps last about half a second
STEP_BYTES_PER_PASS = 4 * (2 + 3) * len(ACTS) * 256 * 256 * 28 * 28


def config_dict():
    """The `config` object: the same in both arms."""
    return {"workload": WORKLOAD, "bytes_per_pass_per_gpu": STEP_BYTES_PER_PASS,
            "passes_per_step": PASSES_PER_STEP,
            "l2": "inputs larger than L2 (205 MB per tensor vs 126 MB), no flush needed",
            "parallelism": "one process per GPU, batch-sharded, no collective on this path"}


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

def _host_threads():
    """Threads the CPU legs use: every core this process may run on (launchers such as
    torch.distributed.run export OMP_NUM_THREADS=1, which would otherwise pin them to one)."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


class CpuPass:
    """The reference's CPU path for one pass (the 8 eltwise ops) over a [n_batch,256,28,28] batch:
    real oneDNN (the build inside PyTorch, through mkldnn tensors) for the three forward activations
    that route exposes, the oracle port (C + OpenMP) for elu forward and the four backward passes.
    Per op it keeps the seconds of the last run."""

    def __init__(self, oracle, n_batch):
        import torch
        self.torch, self.oracle = torch, oracle
        self.threads = _host_threads()
        torch.set_num_threads(self.threads)
        oracle.set_num_threads(self.threads)
        self.shape = [n_batch] + SHAPE_C2[1:]
        self.x = oracle.gen_normal(self.shape, 2.0, 1).reshape(-1)
        self.dy = oracle.gen_normal(self.shape, 1.0, 2).reshape(-1)
        self.y, self.dx = np.empty_like(self.x), np.empty_like(self.x)
        self.n = self.x.size
        self.bytes = self.n * 4 * (2 + 3) * len(ACTS)
        self.mk = None
        try:
            self.mk = torch.from_numpy(self.x).reshape(self.shape).to_mkldnn()
            self.fwd = {"relu": torch.relu, "logistic": torch.sigmoid, "tanh": torch.tanh}
            self.fwd["relu"](self.mk)
        except Exception as e:                       # no mkldnn route: the port does all eight
            self.mk, self.fwd, self.why = None, {}, str(e)[:200]
        self.seconds = {}

    def run(self):
        t_all = time.perf_counter()
        for mode, coef in ACTS:
            t0 = time.perf_counter()
            if mode in self.fwd:
                self.fwd[mode](self.mk)
            else:
                self.oracle.eltwise_fwd(mode, self.x, self.y, coef=coef)
            t1 = time.perf_counter()
            self.oracle.eltwise_bwd(mode, self.x, self.dy, self.dx, coef=coef)
            t2 = time.perf_counter()
            self.seconds[mode + " fwd"] = t1 - t0
            self.seconds[mode + " bwd"] = t2 - t1
        return time.perf_counter() - t_all

    def per_op(self):
        out = {}
        for name, sec in self.seconds.items():
            nbytes = self.n * 4 * (2 if name.endswith("fwd") else 3)
            via = "oneDNN" if name.split()[0] in self.fwd and name.endswith("fwd") else "port"
            out[name] = {"GB/s": round(nbytes / sec / 1e9, 2), "Gelem/s": round(self.n / sec / 1e9, 3), "via": via}
        return out


def onednn_block(n_batch=256, reps=2):
    """Real oneDNN (the build inside PyTorch, through mkldnn tensors) on the host cores for every op of
    the path that route exposes, on the [n_batch,256,28,28] batch: the three forward activations,
    same-shape add / mul and the f32 -> bf16 reorder; GB/s of algorithmic bytes and elements/s.  It has
    no elu, no backward, no broadcast, no reduction and no nhwc reorder: those exist on the CPU only
    as the oracle port."""
    try:
        import torch
        import oracle
        threads = _host_threads()
        torch.set_num_threads(threads)
        shape = [n_batch] + SHAPE_C2[1:]
        n = int(np.prod(shape))
        xd = torch.from_numpy(oracle.gen_normal(shape, 2.0, 1))
        x = xd.to_mkldnn()
        y = torch.from_numpy(oracle.gen_normal(shape, 1.0, 2)).to_mkldnn()
        out = {}
        for name, fn, nbytes in (("relu fwd", lambda: torch.relu(x), n * 8), ("logistic fwd", lambda: torch.sigmoid(x), n * 8),
                                 ("tanh fwd", lambda: torch.tanh(x), n * 8),
                                 ("add (same shape)", lambda: torch.add(x, y), n * 12),
                                 ("mul (same shape)", lambda: torch.mul(x, y), n * 12),
                                 ("reorder f32 -> bf16", lambda: xd.to_mkldnn(torch.bfloat16), n * 6)):
            fn()
            t0 = time.perf_counter()
            for _ in range(reps):
                fn()
            dt = (time.perf_counter() - t0) / reps
            out[name] = {"GB/s": round(nbytes / dt / 1e9, 2), "Gelem/s": round(n / dt / 1e9, 3)}
        ver = [ln.strip(" -") for ln in torch.__config__.show().splitlines() if "MKL-DNN" in ln]
        return {"library": ver[0] if ver else "oneDNN (version unknown)", "threads": threads,
                "sample": "[%d,256,28,28] f32, %d repetitions per op" % (n_batch, reps), "ops": out}
    except Exception as e:  # mkldnn tensors unavailable: report that, the oracle number stands
        return {"unavailable": str(e)[:200]}


def run_reference(args):
    import oracle
    oracle.build()
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cpu = CpuPass(oracle, SHAPE_C2[0])
    for _ in range(args.warmup):
        cpu.run()
    secs = [cpu.run() for _ in range(max(args.steps, 1))]
    t_all = float(np.sum(secs))
    value = cpu.bytes * len(secs) / t_all / 1e9
    sample = ("per step: ONE pass (the 8 eltwise ops) over the full [256,256,28,28] batch, i.e. 1/%d of the GPU arm's "
              "step; GB/s does not depend on the number of passes" % PASSES_PER_STEP)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(1e3 * t_all / len(secs), 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": config_dict(),
        "cpu_baseline": {"value": round(value, 3), "unit": "GB/s", "cores": cpu.threads, "kind": "port",
                         "sample": sample, "per_op": cpu.per_op(),
                         "mix": "relu / tanh / logistic forward through real oneDNN (torch mkldnn tensors), "
                                "elu forward and the four backward passes through oracle/ (C + OpenMP port)"
                                if cpu.mk is not None else "all eight ops through oracle/ (no mkldnn route: %s)" % cpu.why,
                         "onednn": onednn_block()},
        "e2e": {"value": round(value, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference is Clojure on the JVM calling oneDNN; no JVM on this box, so this arm times the "
                "fastest CPU implementation of each op that can run here: real oneDNN where PyTorch exposes the "
                "primitive, the oracle port elsewhere.  One process on the host cores whatever --gpus says.",
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


def ops_table(torch, fact, core, oracle, peak, sharded=None, world=1, profile_only=False, c5_batch=None,
              dist=None, only_sharded_configs=False):
    """Every other configuration's ops, each timed alone: launches captured in a CUDA graph and
    replayed between CUDA events (see graph_ms).  Small tensors rotate through enough distinct
    buffers to exceed L2, so every launch is cold.  With `profile_only` each op is just launched
    three times (a short, fixed launch list for a profiler) and nothing is timed.  With world > 1
    every rank times its own shard and a row holds the slowest rank's time.  `only_sharded_configs`
    keeps the rows that the multi-GPU runs shard (configurations 4 and 5)."""
    rows = []
    h, dev, stream = fact.handle, fact.device, fact.stream
    L2 = 126 << 20
    it = [0]

    def dbuf(nbytes):
        return torch.empty(int(nbytes), dtype=torch.uint8, device=dev)

    def put(arr):
        return torch.from_numpy(np.ascontiguousarray(arr).reshape(-1).view(np.uint8)).to(dev)

    def rotation(nbytes_per_set):
        """How many copies of an op's buffers to rotate through so that a launch never finds its
        input in L2 (1 when one set alone is larger than L2)."""
        return 1 if nbytes_per_set > L2 else max(2, (2 * L2) // nbytes_per_set + 1)

    def measure(name, cfg, nbytes, elems, fn, per_graph, replays, graph=True, rid=None):
        if profile_only:
            for _ in range(3):
                fn()
            stream.synchronize()
            rows.append({"op": name, "config": cfg, "kernel": h.last_kernel()})
            return
        if dist is not None:
            dist.barrier()
        if graph:
            ms = graph_ms(torch, fact, fn, per_graph, replays)
        else:
            ms = event_ms(torch, fn, stream, 100, 10)
        if dist is not None:
            ms = tuple(max_over_ranks(torch, dist, dev, v) for v in ms)
        row = op_row(name, cfg, nbytes, ms, peak, elems)
        row["kernel"] = h.last_kernel()
        if rid:
            row["id"] = rid
        rows.append(row)

    if not only_sharded_configs:
        # C1: fp32 [32,64,56,56] nchw -> nhwc (25.7 MB each way: rotate buffer pairs past L2)
        shp = [32, 64, 56, 56]
        n = int(np.prod(shp))
        xd = core.tensor_descriptor(shp, "float", "nchw")
        yd = core.tensor_descriptor(shp, "float", "nhwc")
        x0 = put(oracle.gen_uniform(shp, -1, 1, 0))
        sets = rotation(n * 8)
        xs = [x0] + [x0.clone() for _ in range(sets - 1)]
        ys = [dbuf(n * 4) for _ in range(sets)]

        def c1():
            i = it[0] % sets
            it[0] += 1
            core.transform_tensor(h, 1.0, xd, xs[i], 0.0, yd, ys[i])

        def c1w():
            core.transform_tensor(h, 1.0, xd, xs[0], 0.0, yd, ys[0])

        def copy_floor():
            i = it[0] % sets
            it[0] += 1
            ys[i].copy_(xs[i])
        measure("reorder f32 nchw->nhwc", "C1 [32,64,56,56], cold L2 (rotating %d buffer pairs)" % sets, n * 8, n, c1, 4 * sets, 20)
        measure("reorder f32 nchw->nhwc (warm L2)", "C1 [32,64,56,56], same buffers every launch", n * 8, n, c1w, 24, 20)
        if not profile_only:
            measure("plain device copy of the same bytes (cudaMemcpyAsync, not this library)",
                    "25.7 MB -> 25.7 MB, same rotation: what a copy reaches at this size in this harness", n * 8, n,
                    copy_floor, 4 * sets, 20)
            rows[-1]["kernel"] = "driver copy (size-matched reference, not a library kernel)"
        del xs, ys

        # C3: broadcast op-tensor on [128,512,14,14]
        shp = [128, 512, 14, 14]
        n = int(np.prod(shp))
        xd = core.tensor_descriptor(shp, "float", "nchw")
        bd = core.tensor_descriptor([1, 512, 1, 1], "float", "nchw")
        bias = put(oracle.gen_uniform([512], -0.1, 0.1, 4))
        scale = put(oracle.gen_uniform([512], 0.5, 1.5, 1004))
        x0 = put(oracle.gen_uniform(shp, -1, 1, 3))
        sets = rotation(n * 8)
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

        def c3copy():
            i = it[0] % sets
            it[0] += 1
            outs[i].copy_(xs[i])
        measure("op-tensor a*x + b*bias[c]", "C3 [128,512,14,14], a=1 b=0.5, cold L2", n * 8 + 2048, n, c3add, 4 * sets, 20)
        measure("op-tensor x * scale[c]", "C3 [128,512,14,14], cold L2", n * 8 + 2048, n, c3mul, 4 * sets, 20)
        if not profile_only:
            measure("plain device copy of the same bytes (cudaMemcpyAsync, not this library)",
                    "51.4 MB -> 51.4 MB, same rotation", n * 8, n, c3copy, 4 * sets, 20)
            rows[-1]["kernel"] = "driver copy (size-matched reference, not a library kernel)"
        del xs, outs

    # C4: reductions on [64,1024,32,32] (268 MB: larger than L2).  With world > 1 each rank holds
    # N/world images (rotated through enough copies to stay out of L2) and the (N,H,W) reductions
    # exchange 4 KB.
    full = [64, 1024, 32, 32]
    shp = [full[0] // world] + full[1:]
    n = int(np.prod(shp))
    xd = core.tensor_descriptor(shp, "float", "nchw")
    x0 = put(oracle.gen_signed_lognormal(shp, 5 + 100 * (sharded.rank if sharded else 0)))
    sets = rotation(n * 4)
    xs = [x0] + [x0.clone() for _ in range(sets - 1)]
    cold = "" if sets == 1 else ", cold L2 (rotating %d copies)" % sets
    for op, yshape, label, rid in (("add", [1, 1024, 1, 1], "sum over (N,H,W)", "c4_sum"),
                                   ("avg", [1, 1024, 1, 1], "mean over (N,H,W)", "c4_mean"),
                                   ("max", [shp[0], 1, 32, 32], "max over C", "c4_max"),
                                   ("norm2", [shp[0], 1, 1, 1], "norm2 over (C,H,W)", "c4_norm2")):
        yd = core.tensor_descriptor(yshape, "float", "nchw")
        y = dbuf(int(np.prod(yshape)) * 4)
        rtd = core.reduce_tensor_descriptor(op, "float")
        spans = sharded is not None and yshape[0] == 1
        nb = n * 4 + int(np.prod(yshape)) * 4
        if spans:
            def fn(rtd=rtd, yd=yd, y=y):
                i = it[0] % sets
                it[0] += 1
                sharded.reduce_tensor(rtd, 1.0, xd, xs[i], 0.0, yd, y, spans=True)
            if sharded.peer_attached:
                sharded.peer_configure(use_peer=True)
                measure("reduce " + label, "C4 shard [%d,1024,32,32]%s + 4 KB exchanged over NVLink by the library's own "
                        "kernels (the form the library picks)" % (shp[0], cold), nb, n, fn, 2 * max(sets, 5), 20, rid=rid)
                if op == "add":
                    def fn_warm(rtd=rtd, yd=yd, y=y):
                        sharded.reduce_tensor(rtd, 1.0, xd, xs[0], 0.0, yd, y, spans=True)
                    if sets > 1:
                        measure("reduce " + label + " (warm L2: the same shard every call)",
                                "C4 shard [%d,1024,32,32] resident in L2" % shp[0], nb, n, fn_warm, 10, 20)
                    for form, kw in (("reduce + exchange in ONE kernel", dict(fused=True)),
                                     ("exchange kernel after the local pass", dict(fused=False))):
                        sharded.peer_configure(use_peer=True, **kw)
                        measure("reduce " + label + " (" + form + ")", "C4 shard [%d,1024,32,32]%s" % (shp[0], cold),
                                nb, n, fn, 2 * max(sets, 5), 20)
                    sharded.peer_configure(use_peer=True)
                sharded.peer_status()
            if op == "add" or not sharded.peer_attached:
                sharded.peer_configure(use_peer=False)
                measure("reduce " + label + " (NCCL)",
                        "C4 shard [%d,1024,32,32]%s + 4 KB ncclAllReduce + finish kernel (un-captured launches)" % (shp[0], cold),
                        nb, n, fn, 10, 20, graph=False, rid=None if sharded.peer_attached else rid)
                sharded.peer_configure(use_peer=True)
        else:
            def fn(rtd=rtd, yd=yd, y=y):
                i = it[0] % sets
                it[0] += 1
                core.reduce_tensor(h, rtd, 1.0, xd, xs[i], 0.0, yd, y)
            measure("reduce " + label, "C4 [%d,1024,32,32]%s" % (shp[0], cold), nb, n, fn, 2 * max(sets, 5), 20, rid=rid)
    del xs, x0

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
    sets = rotation(n * 2)
    qs = [q] + [q.clone() for _ in range(sets - 1)]
    zs = [dbuf(n) for _ in range(sets)]

    def c5s8():
        i = it[0] % sets
        it[0] += 1
        core.transform_tensor(h, 1.0, qd, qs[i], 0.0, zd, zs[i])
    measure("reorder+convert f32 nchw -> bf16 nhwc", "C5 [%d,256,28,28]" % shp[0], n * 6, n,
            lambda: core.transform_tensor(h, 1.0, xd, x, 0.0, yd, y), 5, 10, rid="c5_bf16")
    measure("reorder s8 nchw -> nhwc", "C5 [%d,256,28,28]%s" % (shp[0], "" if sets == 1 else ", cold L2 (rotating %d buffer pairs)" % sets),
            n * 2, n, c5s8, 2 * max(sets, 3), 10, rid="c5_s8")
    del x, y, q, qs, zs

    if not only_sharded_configs and world == 1:
        # reductions away from configuration 4: 16-bit element types, and 784-long runs
        shp = [256, 256, 28, 28]
        n = int(np.prod(shp))
        g = torch.Generator(device=dev)
        g.manual_seed(9)
        xf = torch.randn(n, dtype=torch.float32, device=dev, generator=g)
        for tag, tdt, es in (("float", torch.float32, 4), ("bf16", torch.bfloat16, 2), ("half", torch.float16, 2)):
            xt = xf if tdt == torch.float32 else xf.to(tdt)
            sets = rotation(n * es)        # the 16-bit tensors (103 MB) would otherwise sit in L2
            xts = [xt] + [xt.clone() for _ in range(sets - 1)]
            xd = core.tensor_descriptor(shp, tag, "nchw")
            for op, yshape, label in (("add", [1, 256, 1, 1], "sum over (N,H,W)"), ("max", [256, 1, 28, 28], "max over C")):
                yd = core.tensor_descriptor(yshape, tag, "nchw")
                yb = dbuf(int(np.prod(yshape)) * es)
                rtd = core.reduce_tensor_descriptor(op, "float")

                def fn(rtd=rtd, xd=xd, xts=xts, yd=yd, yb=yb, sets=sets):
                    i = it[0] % sets
                    it[0] += 1
                    core.reduce_tensor(h, rtd, 1.0, xd, xts[i], 0.0, yd, yb)
                measure("reduce " + label + ", " + tag, "[256,256,28,28] %s%s" % (tag, "" if sets == 1 else ", cold L2 (rotating %d copies)" % sets),
                        n * es + int(np.prod(yshape)) * es, n, fn, 2 * max(sets, 3), 10)
            del xt, xts
        one = dbuf(4)
        measure("reduce sum of all elements (what asum / nrm2 / sum of a tensor run)", "[256,256,28,28] float -> 1 value",
                n * 4, n, lambda: core.reduce_tensor(h, core.reduce_tensor_descriptor("add", "float"), 1.0,
                                                     core.tensor_descriptor(shp, "float", "nchw"), xf, 0.0,
                                                     core.tensor_descriptor([1, 1, 1, 1], "float", "nchw"), one), 5, 10)
        del xf
    return rows


def scaling_summary(sharded_rows, full_rows, world):
    """Per sharded configuration: time of the whole tensor on one GPU (measured on rank 0 in this
    run), time per rank on `world` GPUs (slowest rank, collective included), and their ratio."""
    full = {r["id"]: r for r in full_rows if "id" in r}
    out = {"n_gpus": world, "unit": "us per call", "rows": {}}
    for r in sharded_rows:
        rid = r.get("id")
        if rid in full:
            one, many = full[rid]["ms"] * 1e3, r["ms"] * 1e3
            out["rows"][rid] = {"one_gpu": round(one, 2), "per_rank": round(many, 2), "speedup": round(one / many, 2),
                                "frac_of_peak_per_rank": r["frac_of_measured_peak"]}
    return out


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
    # activation kinds of the DNNL backend's table (run-time-switched families): forward and backward
    for mode, coef, shift in (("gelu-tanh", 0.0, 0.0), ("swish", 1.0, 0.0), ("hardswish", 1.0 / 6.0, 0.5)):
        adm = core.activation_descriptor(mode, True, coef, shift)
        measure("%s forward" % mode, "[256,256,28,28] f32", n * 8, n,
                lambda adm=adm: core.activation_forward(h, adm, 1.0, d4, x, 0.0, d4, y))
        measure("%s backward" % mode, "[256,256,28,28] f32", n * 12, n,
                lambda adm=adm: core.activation_backward(h, adm, 1.0, d4, None, d4, z, d4, x, 0.0, d4, y))
    # oneDNN's norm-lp-sum with p = 3 over (C,H,W): |x|^p element by element
    rl = core.reduce_tensor_descriptor("norm-lp-sum", "float", True, p=3.0, eps=1e-6)
    yl = torch.empty(256, dtype=torch.float32, device=dev)
    measure("reduce norm-lp-sum p=3 over (C,H,W)", "[256,256,28,28] f32", n * 4, n,
            lambda: core.reduce_tensor(h, rl, 1.0, d4, x, 0.0, core.tensor_descriptor([256, 1, 1, 1], "float", "nchw"), yl))
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
    del z

    # the late stages of a CNN: 7 x 7 maps, whose rows of 49 elements are not whole 16-byte vectors
    s7 = [1024, 1024, 7, 7]
    n7 = int(np.prod(s7))                       # as many elements as [256,256,28,28]
    d7 = core.tensor_descriptor(s7, "float", "nchw")
    d7h = core.tensor_descriptor(s7, "float", "nhwc")
    bias7 = torch.randn(1024, dtype=torch.float32, device=dev, generator=g)
    db7 = core.tensor_descriptor([1, 1024, 1, 1], "float", "nchw")
    measure("bias add on 7x7 maps", "[1024,1024,7,7] f32 nchw", n7 * 8, n7,
            lambda: core.op_tensor(h, "add", 1.0, d7, x, 1.0, db7, bias7, 0.0, d7, y))
    gb7 = torch.zeros(1024, dtype=torch.float32, device=dev)
    measure("bias gradient (sum over N,H,W) on 7x7 maps", "[1024,1024,7,7] f32 nchw", n7 * 4, n7,
            lambda: core.convolution_bwd_bias(h, 1.0, d7, x, 0.0, db7, gb7))
    mx7 = torch.zeros(1024 * 49, dtype=torch.float32, device=dev)
    rmax = core.reduce_tensor_descriptor("max", "float")
    dm7 = core.tensor_descriptor([1024, 1, 7, 7], "float", "nchw")
    measure("max over C on 7x7 maps", "[1024,1024,7,7] f32 nchw", n7 * 4, n7,
            lambda: core.reduce_tensor(h, rmax, 1.0, d7, x, 0.0, dm7, mx7))
    measure("reorder nchw -> nhwc on 7x7 maps", "[1024,1024,7,7] f32", n7 * 8, n7,
            lambda: core.transform_tensor(h, 1.0, d7, x, 0.0, d7h, y))
    measure("reorder nhwc -> nchw on 7x7 maps", "[1024,1024,7,7] f32", n7 * 8, n7,
            lambda: core.transform_tensor(h, 1.0, d7h, x, 0.0, d7, y))
    s7b = [2048, 2048, 7, 7]
    n7b = int(np.prod(s7b))                     # 205 MB of int8, the bytes of x
    d7b = core.tensor_descriptor(s7b, "byte", "nchw")
    d7bh = core.tensor_descriptor(s7b, "byte", "nhwc")
    measure("reorder int8 nchw -> nhwc on 7x7 maps", "[2048,2048,7,7] s8", n7b * 2, n7b,
            lambda: core.transform_tensor(h, 1.0, d7b, x, 0.0, d7bh, y))
    # a batch of images as a loader hands them over (uint8, channels last) into the f32 nchw tensor a
    # network reads: 3 channels, too thin for a tile
    simg = [336, 3, 224, 224]
    nimg = int(np.prod(simg))                   # 50.6 M elements: 50.6 MB in, 202 MB out
    measure("uint8 nhwc images -> f32 nchw", "[336,3,224,224]", nimg * 5, nimg,
            lambda: core.transform_tensor(h, 1.0, core.tensor_descriptor(simg, "uint8", "nhwc"), x, 0.0,
                                          core.tensor_descriptor(simg, "float", "nchw"), y))
    measure("f32 nchw -> nhwc, 3 channels", "[336,3,224,224]", nimg * 8, nimg,
            lambda: core.transform_tensor(h, 1.0, core.tensor_descriptor(simg, "float", "nchw"), x, 0.0,
                                          core.tensor_descriptor(simg, "float", "nhwc"), y))
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
    elif args.profile_shard:
        # what ONE of 8 GPUs holds of configurations 4 and 5 ([8,1024,32,32], [256,256,28,28]),
        # reduced / reordered locally
        rows = ops_table(torch, fact, core, oracle, peaks()[0], None, 8, profile_only=True, only_sharded_configs=True)
    else:
        rows = ops_table(torch, fact, core, oracle, peaks()[0], None, 1, profile_only=True, c5_batch=256)
    print(json.dumps({"profile_ops": rows}))
    fact.release()


# ------------------------------------------------------------------ main GPU arm ---------------

def bind_near_gpu(cuda_index):
    """Pins this process to the CPUs of the NUMA node the GPU hangs off (read-only look-ups in sysfs),
    BEFORE any pinned host buffer is allocated: page-locked memory is then taken from that node, and
    host <-> device copies do not cross the socket interconnect.  Returns what it found and did."""
    info = {"numa_node": None, "bound": False}
    try:
        import pynvml
        import torch
        pynvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(cuda_index).uuid)
        hd = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid if not uuid.startswith("GPU-") else uuid).encode())
        bus = pynvml.nvmlDeviceGetPciInfo(hd).busId
        bus = bus.decode() if isinstance(bus, bytes) else bus
        bdf = bus.lower()[-12:]                                   # 0000:1b:00.0
        with open("/sys/bus/pci/devices/%s/numa_node" % bdf) as f:
            node = int(f.read().strip())
        info["numa_node"] = node
        if node < 0:
            return info
        with open("/sys/devices/system/node/node%d/cpulist" % node) as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0) & cpus
        info["node_cpus_allowed"] = len(allowed)
        if allowed:
            os.sched_setaffinity(0, allowed)
            info["bound"] = True
    except Exception as e:
        info["error"] = str(e)[:120]
    return info


def max_over_ranks(torch, dist, device, value):
    if dist is None:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sharded_parity(torch, dist, fact, core, oracle, sh, world, rank):
    """Before anything sharded is timed: the reductions that fold the sharded batch, on every combine
    path, against the oracle's reduction of the WHOLE tensor (rank 0 builds it from the ranks' seeds
    and broadcasts the expected results), plus bit-equality of the replicated results across ranks.
    Bar: |got - want| <= max(1e-5 |want|, 16 u sum|x|) (pairwise fp32 summation of signed log-normal
    data: the second term is the conditioning floor); max is bit-exact."""
    nb = 64 // world
    shp = [nb, 1024, 32, 32]
    mine = oracle.gen_signed_lognormal(shp, 5 + 100 * rank)
    x = torch.from_numpy(mine).to(fact.device)
    xd = core.tensor_descriptor(shp, "float", "nchw")
    yshape = [1, 1024, 1, 1]
    yd = core.tensor_descriptor(yshape, "float", "nchw")
    ops = ("add", "avg", "norm2", "max")
    want = torch.zeros(len(ops) + 1, 1024, dtype=torch.float64)
    if rank == 0:
        full = np.concatenate([mine] + [oracle.gen_signed_lognormal(shp, 5 + 100 * r) for r in range(1, world)])
        for i, op in enumerate(ops):
            w = np.zeros(yshape, np.float32)
            oracle.reduce(op, full, w)
            want[i] = torch.from_numpy(w.reshape(-1).astype(np.float64))
        want[len(ops)] = torch.from_numpy(np.abs(full.astype(np.float64)).sum(axis=(0, 2, 3)))
        del full
    want = want.to(fact.device)
    dist.broadcast(want, src=0)
    want = want.cpu().numpy()
    scale = want[len(ops)]
    out = {"tensor": "[64,1024,32,32] signed log-normal, %d images per rank" % nb, "paths": {}}
    paths = [("fused", dict(use_peer=True, fused=True)), ("separate", dict(use_peer=True, fused=False)),
             ("nccl", dict(use_peer=False))] if sh.peer_attached else [("nccl", dict(use_peer=False))]
    ok = True
    for pname, kw in paths:
        sh.peer_configure(**kw)
        entry = {}
        for i, op in enumerate(ops):
            y = torch.zeros(1024, dtype=torch.float32, device=fact.device)
            sh.reduce_tensor(core.reduce_tensor_descriptor(op, "float"), 1.0, xd, x, 0.0, yd, y, spans=True)
            fact.synchronize()
            got = y.cpu().numpy().astype(np.float64)
            gathered = [torch.zeros_like(y) for _ in range(world)]
            dist.all_gather(gathered, y)
            same = all(torch.equal(gathered[0], g) for g in gathered)
            err = np.abs(got - want[i])
            if op == "max":
                good = bool(np.array_equal(got, want[i]))
                entry[op] = {"bit_exact": good, "replicas_identical": same}
            else:
                div = {"add": 1.0, "avg": float(64 * 1024), "norm2": 1.0}[op]
                floor = 16 * 6e-8 * scale / div if op != "norm2" else 16 * 6e-8 * np.abs(want[i])
                bound = np.maximum(1e-5 * np.abs(want[i]), floor)
                good = bool((err <= bound).all())
                entry[op] = {"max_rel_err": float(np.max(err / np.maximum(np.abs(want[i]), 1e-300))),
                             "channels_within_1e-5": int((err <= 1e-5 * np.abs(want[i])).sum()),
                             "channels_needing_the_floor": int(((err > 1e-5 * np.abs(want[i])) & (err <= bound)).sum()),
                             "channels_outside": int((err > bound).sum()), "replicas_identical": same}
            ok = ok and good and same
        out["paths"][pname] = entry
    if sh.peer_attached:
        sh.peer_configure(use_peer=True)
        sh.peer_status()
    flag = torch.tensor([0 if ok else 1], device=fact.device)
    dist.all_reduce(flag)
    out["ok"] = int(flag.item()) == 0
    del x
    return out


def run_ours(args):
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    host_binding = bind_near_gpu(local_rank) if world > 1 else {"bound": False, "note": "one rank: left unbound"}
    dist = None
    # stdout carries ONE JSON line: whatever libraries print there meanwhile (NCCL announces its
    # version on stdout at the first communicator) goes to stderr instead
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")  # keep stdout to the one JSON line
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    import oracle
    from deep_diamond_b200 import b200_factory, core, dnn, sharded as shd, tensor as T
    if rank == 0:
        oracle.build()
    if dist:
        dist.barrier()
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
    pass_bytes = len(ACTS) * (fwd_bytes + bwd_bytes)
    assert pass_bytes == STEP_BYTES_PER_PASS

    def one_pass(events=None):
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
        for _ in range(PASSES_PER_STEP):
            one_pass()
    stream.synchronize()
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = h.launch_count()
    events = []
    t_start, t_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t_start.record(stream)
    for _ in range(args.steps):
        for j in range(PASSES_PER_STEP):
            one_pass(events if j == PASSES_PER_STEP // 2 else None)   # one pass per step timed launch by launch
    t_stop.record(stream)
    stream.synchronize()
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    if dist:
        dist.barrier()
    launches = h.launch_count() - launches0
    total_ms = max_over_ranks(torch, dist, fact.device, t_start.elapsed_time(t_stop))
    if clocks is not None:
        clocks["window"] = "the timed region (%d steps x %d passes, %.0f ms)" % (args.steps, PASSES_PER_STEP, total_ms)

    fwd_ms = {m: [] for m, _ in ACTS}
    bwd_ms = {m: [] for m, _ in ACTS}
    pass_ms = []
    for i in range(0, len(events), len(ACTS)):
        grp = events[i:i + len(ACTS)]
        pass_ms.append(grp[0][1].elapsed_time(grp[-1][3]))
        for m, e0, e1, e2 in grp:
            fwd_ms[m].append(e0.elapsed_time(e1))
            bwd_ms[m].append(e1.elapsed_time(e2))
    value = world * args.steps * PASSES_PER_STEP * pass_bytes / (total_ms * 1e-3) / 1e9
    burst = world * pass_bytes / (max_over_ranks(torch, dist, fact.device, min(pass_ms)) * 1e-3) / 1e9
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
        parity = {"elu_fwd_max_ulp": int(oracle.ulp_diff_f32(got_y, want_y).max()),
                  "elu_bwd_max_ulp": int(oracle.ulp_diff_f32(got_dx, want_dx).max()), "checked_elements": k}

    # End to end through the public API with pinned HOST buffers.  Per step: x and dy go up ONCE
    # each, the four layers run forward + backward (each layer's upstream gradient is a device-side
    # copy of dy into its diff-input buffer, as the next layer of a network would leave it there),
    # y of the logistic layer and dx of the last layer come back.  Uploads and downloads run on
    # separate copy streams, so the read-back of a step overlaps the upload of the next.
    tz_x = T.tensor(fact, SHAPE_C2, "float", "nchw")
    tz_dx = T.tensor(fact, SHAPE_C2, "float", "nchw")
    tz_dy = T.tensor(fact, SHAPE_C2, "float", "nchw")
    pin_x = torch.from_numpy(x_host).pin_memory()
    pin_dy = torch.from_numpy(dy_host).pin_memory()
    pin_y = torch.empty(n, dtype=torch.float32).pin_memory()
    pin_dx = torch.empty(n, dtype=torch.float32).pin_memory()
    layers = [dnn.activation(fact, tz_x, m, {"alpha": c})(tz_x, tz_dx) for m, c in ACTS]
    logistic = [l for l, (m, _) in zip(layers, ACTS) if m == "logistic"][0]
    pend = {"y": None, "dx": None}

    def e2e_step():
        T.transfer_async(pin_x.numpy(), tz_x)
        T.transfer_async(pin_dy.numpy(), tz_dy)
        for layer in layers:
            if layer is logistic and pend["y"] is not None:
                pend["y"].before_overwrite()          # last step's y is still being read from this buffer
            layer.forward()
            if layer is logistic:
                pend["y"] = T.transfer_async(layer.output(), pin_y.numpy())
            T.transfer(tz_dy, layer.diff_input())     # device -> device, on the compute stream
            if layer is layers[0] and pend["dx"] is not None:
                pend["dx"].before_overwrite()         # every backward writes the shared dx
            layer.backward()
        pend["dx"] = T.transfer_async(tz_dx, pin_dx.numpy())

    def e2e_drain():
        for p in pend.values():
            if p is not None:
                p.wait()

    e2e_steps = 0 if args.no_e2e else max(1, min(args.steps, 20))
    e2e = None
    if e2e_steps:
        e2e_step()
        e2e_drain()
        torch.cuda.synchronize()
        # each direction alone, for the record: one upload and one download of a 205 MB tensor
        t0 = time.perf_counter()
        T.transfer_async(pin_x.numpy(), tz_x)
        fact.synchronize()
        torch.cuda.synchronize()
        up_s = time.perf_counter() - t0
        t0 = time.perf_counter()
        T.transfer_async(tz_dx, pin_dx.numpy()).wait()
        down_s = time.perf_counter() - t0
        if dist:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        e2e_drain()
        torch.cuda.synchronize()
        e2e_s = max_over_ranks(torch, dist, fact.device, (time.perf_counter() - t0) / e2e_steps)
        h2d, d2h = n * 4 * 2, n * 4 * 2
        e2e = {"value": round(world * pass_bytes / e2e_s / 1e9, 2), "unit": "GB/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_s * 1e3, 3),
               "steps": e2e_steps, "work_per_step": "one pass (the 8 ops) over the batch",
               "h2d_GB/s_in_step": round(h2d / e2e_s / 1e9, 1), "d2h_GB/s_in_step": round(d2h / e2e_s / 1e9, 1),
               "h2d_GB/s_alone": round(n * 4 / up_s / 1e9, 1), "d2h_GB/s_alone": round(n * 4 / down_s / 1e9, 1),
               "host_memory_traffic_GB/s_all_ranks": round(world * (h2d + d2h) / e2e_s / 1e9, 1),
               "host": host_binding,
               "api": "tensor.transfer_async (pinned numpy <-> device, uploads and downloads on separate copy "
                      "streams), tensor.transfer (device -> device), dnn.activation layers forward/backward"}
        if rank == 0:
            # what came back over the pipelined copies: y = logistic(x), dx = elu'(x) * dy (the last layer)
            k = 1 << 16
            wy = oracle.eltwise_fwd("logistic", x_host[:k], np.empty(k, np.float32))
            wdx = oracle.eltwise_bwd(ACTS[-1][0], x_host[:k], dy_host[:k], np.empty(k, np.float32), coef=ACTS[-1][1])
            e2e["result_max_ulp"] = {"y": int(oracle.ulp_diff_f32(pin_y.numpy()[:k], wy).max()),
                                     "dx": int(oracle.ulp_diff_f32(pin_dx.numpy()[:k], wdx).max())}
    del layers, tz_x, tz_dx, tz_dy, pin_x, pin_dy, pin_y, pin_dx

    ops = ops_next = shard_par = summary = None
    if not args.no_ops:
        del x, dy, y, dx
        torch.cuda.empty_cache()
        sh = None
        if world > 1:
            sh = shd.create_from_torch_distributed(fact)
            shard_par = sharded_parity(torch, dist, fact, core, oracle, sh, world, rank)
        ops = ops_table(torch, fact, core, oracle, peak, sh, world, dist=dist)
        if sh is not None:
            sh.release(barrier=dist.barrier)
        torch.cuda.empty_cache()
        if world > 1:
            # the same ops on the WHOLE tensors on one GPU, in the same run (rank 0 only), for the
            # strong-scaling ratios of the sharded configurations
            full = ops_table(torch, fact, core, oracle, peak, None, 1, only_sharded_configs=True) if rank == 0 else []
            dist.barrier()
            summary = scaling_summary(ops, full, world) if rank == 0 else None
        ops_next = next_rows_table(torch, fact, core, oracle, peak) if world == 1 else None

    cpu = None
    if rank == 0 and world == 1:
        cp = CpuPass(oracle, SHAPE_C2[0])
        cp.run()
        secs = [cp.run() for _ in range(3)]
        gbs = cp.bytes * len(secs) / float(np.sum(secs)) / 1e9
        onednn = onednn_block()
        if "ops" in onednn:
            for name, gkey in (("relu fwd", ("relu", "fwd_GB/s")), ("logistic fwd", ("logistic", "fwd_GB/s")),
                               ("tanh fwd", ("tanh", "fwd_GB/s"))):
                onednn["ops"][name]["gpu_over_onednn"] = round(per_kernel[gkey[0]][gkey[1]] / onednn["ops"][name]["GB/s"], 1)
        cpu = {"value": round(gbs, 3), "unit": "GB/s", "cores": cp.threads, "kind": "port",
               "gpu_over_cpu": round(value / gbs, 1),
               "sample": "one pass (the 8 eltwise ops) over the full [256,256,28,28] batch, 3 repetitions",
               "mix": "relu / tanh / logistic forward through real oneDNN (torch mkldnn tensors), elu forward and the "
                      "four backward passes through oracle/ (C + OpenMP port)" if cp.mk is not None else
                      "all eight ops through oracle/",
               "per_op": cp.per_op(), "onednn": onednn}

    if rank == 0:
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(total_ms / args.steps, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": config_dict(),
            "sustained_vs_burst": {"sustained_GB/s": round(value, 1), "timed_region_ms": round(total_ms, 1),
                                   "burst_GB/s": round(burst, 1),
                                   "burst_is": "the fastest of the %d passes (8 launches each) that were timed launch by "
                                               "launch; the event records between its launches cost it a few per cent, "
                                               "which is why it can read below the sustained figure" % len(pass_ms)},
            "frac_of_measured_peak": round(value / world / peak, 4),
            "roofline": {"bound": "hbm", "kernel": "activation backward: dd_elt_flat_kernel<float,float,relu,BWD> and dd_elt_flat_multi_kernel<tanh|logistic|elu,BWD,2>",
                         "achieved": round(achieved, 1), "peak": peak, "peak_kind": "of " + peak_kind, "unit": "GB/s",
                         "frac": round(achieved / peak, 4), "frac_of_nominal_8TBs": round(achieved / NOMINAL_HBM_GBS, 4),
                         "traffic": TRAFFIC_BWD["bytes"], "traffic_source": TRAFFIC_BWD,
                         "avg_launch_ms": round(bwd_avg_ms, 5), "launches_timed": len(all_bwd),
                         "algorithmic_bytes_per_launch": bwd_bytes},
            "per_kernel": per_kernel,
            "cpu_baseline": cpu,
            "e2e": e2e,
            "gpu_launches": int(launches),
            "clocks": clocks,
            "parity_spot_check": parity,
            "ops": ops,
            "ops_next": ops_next,
            "sharded_parity": shard_par,
            "scaling_summary": summary,
        }
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        print(json.dumps(line), flush=True)
        os.dup2(2, 1)
    fact.release()
    if dist:
        dist.destroy_process_group()
    sys.stdout.flush()
    os.dup2(real_stdout, 1)


def main():
    global PASSES_PER_STEP
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-ops", action="store_true", help="skip the per-op table of the other configurations")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg (for profiler captures)")
    ap.add_argument("--profile-next", action="store_true",
                    help="like --profile-ops for the table of the path's callers (shuffler, branch, sum, cost ...)")
    ap.add_argument("--profile-shard", action="store_true",
                    help="like --profile-ops for the per-GPU shards of configurations 4 and 5 at 8 GPUs")
    ap.add_argument("--passes", type=int, default=0,
                    help="passes per step (default %d); 1 keeps a profiler capture short" % PASSES_PER_STEP)
    ap.add_argument("--profile-ops", action="store_true",
                    help="launch each op of the per-op table three times and exit (for profiler captures)")
    args = ap.parse_args()
    if args.passes > 0:
        PASSES_PER_STEP = args.passes
    if args.profile_ops or args.profile_next or args.profile_shard:
        run_profile_ops(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
