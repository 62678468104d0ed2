#!/usr/bin/env python
"""Benchmark of the MixedQLinear hot path on B200.

One step = one pass of the four linear layers of a Llama-2 decoder layer (fused-N shapes: qkv,
o, gate+up int4 with 256 fp16 outlier columns, down int8) over M tokens of seeded synthetic
activations: activation quantizer + fused int GEMM / outlier GEMM / dequantize per layer.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--model 70b|7b] [--tokens M] [--dtype fp16|bf16]
                    [--impl reference] [--config 0|1|3|4|all]

Default workload: the Llama-2-70B shapes at M = 4096 (the configuration named for 1/2/4/8 GPUs); on one
GPU the same JSON line also carries `secondary_7b` (the 7B shapes at M = 2048 with their own roofline),
`small_m` (the 7B shapes at M = 16, HBM-bound) and `decoder_block`.

Prints one JSON line (rank 0).  `value` is whole-job TOPS (2*M*N*K summed over the layers / time)
with inputs resident in HBM; `e2e` is the same metric through MixedQLinear.forward with the
activations copied from pinned host memory and the outputs copied back inside the timed region.
N > 1 (torchrun): the layers are column-sharded over the ranks and the outputs assembled on every rank.
`--impl reference` times the reference's torch fake-quant simulation of the same layers on the
host cores (a port of it; the reference checkout is not needed at run time).
`--config` times the layers of one of the benchmark configurations one by one and prints a table.

Timing: after W (>= 3) warm-up steps the K-step loop is repeated back to back until at least
`--min-seconds` of device time has passed, with a CUDA event between repetitions; `ms_per_step` is the median
repetition (max over ranks) divided by K, so the figure is a sustained one and the clock samples fall inside the load.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "MixedQLinear TOPS (Llama-2 linear shapes, fused quantize+GEMM+dequant)"
L2_BYTES = 126e6
# dram__bytes_read.sum + dram__bytes_write.sum per launch of gemm_tcgen05_kernel from `ncu --set full` captures of
# single bench steps, key = (M, K, N); the files under profiles/ named here hold the captures' figures and commands
NCU_TRAFFIC_BYTES = {
    (2048, 4096, 12288): 84.55e6, (2048, 4096, 4096): 26.88e6, (2048, 4096, 22016): 178.77e6, (2048, 11008, 4096): 84.54e6,
}
NCU_TRAFFIC_SOURCE = "profiles/gemm_tcgen05_llama7b_m2048.md"
# The 70B layers at M = 4096 hold up to 1.3 GB per launch, more than a full-section capture should; one layer of them
# was captured (o, 8192 -> 8192: 281.0 MB of DRAM traffic for 266.6 MB of algorithmic bytes) and the others are scaled
# from it by their algorithmic bytes (operands and outputs cross HBM once in every layer: traffic grows in proportion).
NCU_TRAFFIC_RATIO_70B = 281.0 / 266.6
NCU_TRAFFIC_RATIO_SOURCE = ("profiles/gemm_tcgen05_llama70b_m4096.md (capture of the o layer; the other layers scaled "
                            "by algorithmic bytes)")


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--tokens", type=int, default=0, help="default: 4096 for the 70b shapes, 2048 for the 7b shapes")
    ap.add_argument("--model", choices=["7b", "70b"], default="70b")
    ap.add_argument("--dtype", choices=["fp16", "bf16"], default="fp16", help="type of activations and outputs")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--config", default="", help="time one benchmark configuration layer by layer: 0, 1, 3, 4 or all")
    ap.add_argument("--engine", choices=["auto", "tcgen05", "mma_sync"], default="auto")
    ap.add_argument("--tile-n", type=int, default=0)
    ap.add_argument("--l2-hint", type=int, default=-1, help="override QUIK_CFG_L2_HINT (0 / 1)")
    ap.add_argument("--stream-preload", type=int, default=-1, help="override QUIK_CFG_STREAM_PRELOAD (0 / 1)")
    ap.add_argument("--stream-ring", type=int, default=-1, help="override QUIK_CFG_STREAM_RING (0 / 1 / 2)")
    ap.add_argument("--small-m-engine", type=int, default=-1,
                    help="override QUIK_CFG_SMALL_M (0 off, 1 by layer size, 2 direct loads, 3 tcgen05 ring, 4 mma.sync ring)")
    ap.add_argument("--min-seconds", type=float, default=1.0, help="least device time of the timed region")
    ap.add_argument("--no-library-peak", action="store_true",
                    help="do not time the cuBLASLt int8 GEMM (keeps a profiler's launch list to this repository's kernels)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="skip secondary_7b, small_m and decoder_block")
    ap.add_argument("--layers", default="", help="comma-separated subset of layer names")
    ap.add_argument("--no-graph", action="store_true",
                    help="time eager launches instead of replaying the step as a CUDA graph")
    ap.add_argument("--tp-chunks", type=int, default=1,
                    help="N > 1, pull mode: row blocks per layer forward (0: by the size of the output)")
    ap.add_argument("--tp-copy", choices=["auto", "ce", "sm"], default="ce",
                    help="N > 1, pull mode: copy engines, the copy kernel, or the kernel for short rows only")
    ap.add_argument("--tp-mode", choices=["pull", "nccl"], default="pull",
                    help="N > 1: assemble outputs by peer copies out of symmetric memory, or by NCCL all-gather")
    args = ap.parse_args()
    if args.tokens <= 0:
        args.tokens = 4096 if args.model == "70b" else 2048
    return args


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained") or p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs (a read-only query)."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.lines = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self, window=None):
        """window = (t0, t1) in time.perf_counter() seconds: only samples taken inside it count."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.1)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, ln in self.lines:
            if window is not None and not (window[0] <= t <= window[1]):
                continue
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_min_mhz": min(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None, "power_w_median": statistics.median(power) if power else None,
                "samples": len(sm), "reasons": sorted(reasons),
                "window": "samples taken between the first and the last launch of the timed region"}


def measure_library_int8(dev):
    """cuBLASLt int8 GEMM (torch._int_mm) at 8192^3, outside any timed region: best of 10 (burst) and two seconds back to
    back (sustained).  The measured-peak file holds HBM and bf16 figures only; this anchors the int8 tensor peak."""
    try:
        n = 8192
        a = torch.randint(-128, 127, (n, n), dtype=torch.int8, device=dev)
        b = torch.randint(-128, 127, (n, n), dtype=torch.int8, device=dev)
        for _ in range(3):
            torch._int_mm(a, b.t())
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._int_mm(a, b.t())
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        burst = 2.0 * n ** 3 / (best * 1e-3) / 1e12
        reps = max(20, int(2.0 / (best * 1e-3)))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            torch._int_mm(a, b.t())
        e1.record()
        torch.cuda.synchronize()
        sustained = reps * 2.0 * n ** 3 / (e0.elapsed_time(e1) * 1e-3) / 1e12
        del a, b
        torch.cuda.empty_cache()
        return {"burst": burst, "sustained": sustained}
    except Exception as exc:  # pragma: no cover - depends on the library build
        return {"error": str(exc)[:160]}


def int8_peaks(peaks, lib_int8):
    """The int8 tensor peak for a kernel timed alone (burst) and inside a long region (sustained): the larger of the
    measured library int8 GEMM and twice the measured bf16 GEMM (int8 runs at twice the bf16 rate on this part)."""
    out = {}
    for kind, bf in (("burst", peaks["bf16_tflops"]), ("sustained", peaks["bf16_tflops_sustained"])):
        cands = {f"2 x bf16 {kind} GEMM peak of {peaks['source']} ({bf} TF/s)": 2.0 * bf}
        if lib_int8 and kind in lib_int8:
            cands[f"cuBLASLt int8 GEMM 8192^3 measured in this run, {kind}"] = lib_int8[kind]
        src = max(cands, key=cands.get)
        out[kind] = (cands[src], src)
    return out


# ---------------------------------------------------------------------------------------------
def cpu_fake_quant_layers(shapes, tokens, seed=0):
    """The layers of the step as the reference's torch fake-quant simulation (experiments/quant_sim.py ActQuantWrapper
    around nn.Linear with RTN-quantized weights), ported in oracle/fakequant.py, with their seeded inputs."""
    from oracle import fakequant
    from quik_b200 import workloads
    torch.set_num_threads(os.cpu_count() or 1)
    layers = []
    ops = 0.0
    for (name, K, N, bits) in shapes:
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(tokens, K, generator=g)
        fp_idx = torch.randperm(K, generator=g)[:workloads.FP_FEATURES]
        x[:, fp_idx] *= 20
        w = (0.02 * torch.randn(N, K, generator=g)).half()
        standin = workloads.standin_act_scales(K, fp_idx)
        layer = fakequant.FakeQuantLinear(w, standin, workloads.FP_FEATURES, bits)
        # weight fake-quantization is a one-off preparation step; plain RTN keeps the set-up short
        wi = w[:, layer.q_idx].float()
        sc = fakequant.weight_rtn_params(wi, bits, clip=False)
        w[:, layer.q_idx] = fakequant.weight_rtn_quantize(wi, sc, bits).half()
        del wi
        layer.weight = w
        layers.append((layer, x.half()))
        ops += 2.0 * tokens * N * K
    return layers, ops


def cpu_fake_quant_time(layers, ops, tokens, steps, warmup):
    """Times `steps` passes over the layers on the host cores after `warmup` passes."""
    times = []
    with torch.no_grad():
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            for layer, x in layers:
                layer(x)
            dt = time.perf_counter() - t0
            if i >= warmup:
                times.append(dt)
    mean = sum(times) / len(times)
    return {"value": ops / mean / 1e12, "unit": "TOPS", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"all {tokens} tokens of the workload per layer, all {len(layers)} layers, "
                      f"{steps} timed passes after {warmup} warm-up (oracle/fakequant.py on "
                      f"{os.cpu_count()} host cores)", "ms_per_step": mean * 1e3}


def run_reference_arm(args, shapes, config):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # one pass over the full workload is seconds of CPU work: the arm keeps the GPU arm's warm-up and step counts as
    # long as the whole run stays within about four minutes, else it shortens them and says so in `sample`
    layers, ops = cpu_fake_quant_layers(shapes, args.tokens)
    probe = cpu_fake_quant_time(layers, ops, args.tokens, 1, 1)
    per_pass = probe["ms_per_step"] * 1e-3
    budget = 240.0
    want_warm = max(args.warmup, 3)
    warm = max(1, min(want_warm, int(budget * 0.2 / per_pass)))
    steps = max(1, min(args.steps, int(budget * 0.8 / per_pass)))
    base = cpu_fake_quant_time(layers, ops, args.tokens, steps, warm)
    if steps < args.steps or warm < want_warm:
        base["sample"] += f"; shortened from {args.steps} steps / {want_warm} warm-up to stay within a few minutes"
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": "TOPS", "n_gpus": args.gpus,
            "steps": steps, "warmup": warm, "ms_per_step": base["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic", "config": config,
            "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": base["value"], "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
class Workload:
    """The layers of one benchmark step on this rank, and how to run them."""

    def __init__(self, shapes, M, dev, dtype, world=1, rank=0, tp_mode="pull", copies=1, tp_chunks=None, tp_copy="ce"):
        from quik_b200 import workloads
        from quik_b200.tp import ColumnParallelMixedQLinear, shard_range
        self.shapes, self.M, self.world, self.dev = shapes, M, world, dev
        self.cases, self.layers = [], []
        for (name, K, N, bits) in shapes:
            sl = shard_range(N, world, rank) if world > 1 else None
            c = workloads.make_layer(name, M, K, N, bits, seed=0, device=dev, dtype=dtype, n_slice=sl)
            self.cases.append(c)
            self.layers.append(ColumnParallelMixedQLinear(c.module, mode=tp_mode, chunks=tp_chunks, copy=tp_copy) if world > 1 else c.module)
            torch.cuda.empty_cache()
        self.total_ops = sum(2.0 * M * N * K for (_, K, N, _) in shapes)           # whole job, all ranks
        self.alg_bytes = sum(c.algorithmic_bytes for c in self.cases)
        # further copies of the modules (same values, other addresses): a step then walks over `copies` sets of
        # weights in turn so that weights are not served from L2 when one set alone would fit there
        self.sets = [self.layers]
        if copies > 1 and world == 1:
            import copy
            for _ in range(copies - 1):
                self.sets.append([copy.deepcopy(layer) for layer in self.layers])
        self.graph = None
        self._turn = 0
        # tensor parallel: a graph holds an even number of steps (the assembled results alternate between two
        # buffers); inside it the assembly of a step overlaps the kernels of the following steps
        self.graph_steps = 4 if world > 1 else len(self.sets)

    def step(self, wait=True):
        layers = self.sets[self._turn % len(self.sets)]
        self._turn += 1
        outs = [layer(c.x.unsqueeze(0)) for c, layer in zip(self.cases, layers)]
        if self.world > 1 and wait:
            for layer in layers:
                layer.wait()          # the assembled outputs are part of the step
        return outs

    def reset(self):
        for layers in self.sets:
            for layer in layers:
                if hasattr(layer, "reset"):
                    layer.reset()

    def capture(self, sync_all, rank):
        """The step as a CUDA graph (the launches are replayed without host work in between); with several weight
        sets one graph holds one step per set.  Falls back to eager launches if capture fails."""
        try:
            self.reset()
            self._turn = 0
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                # only the last step joins the assembly streams: every output is complete when the graph ends
                self.graph_outs = [self.step(wait=(i == self.graph_steps - 1)) for i in range(self.graph_steps)]
            self.graph = g
            for _ in range(3):
                g.replay()
            sync_all()
        except Exception as exc:  # pragma: no cover - depends on the runtime
            if rank == 0:
                print(f"# CUDA graph capture failed, timing eager launches: {exc}", file=sys.stderr)
            self.graph = None
            sync_all()

    @property
    def steps_per_run(self):
        return self.graph_steps if self.graph is not None else 1

    def run(self):
        if self.graph is not None:
            self.graph.replay()
        else:
            self.step()


def timed_region(wl, steps, min_seconds, sync_all, world, dev):
    """K steps per repetition, repetitions back to back until `min_seconds` of device time, CUDA events between
    repetitions, barrier + synchronize on both sides, max over ranks per repetition."""
    import torch.distributed as dist
    runs = max(1, math.ceil(steps / wl.steps_per_run))          # graph replays per repetition
    k = runs * wl.steps_per_run                                 # steps per repetition (= steps unless weight sets rotate)
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(runs):
        wl.run()
    e1.record()
    sync_all()
    est = torch.tensor([e0.elapsed_time(e1) * 1e-3], device=dev)
    if world > 1:
        dist.all_reduce(est, op=dist.ReduceOp.MAX)
    reps = int(min(400, max(3, math.ceil(min_seconds / max(est.item(), 1e-6)))))
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
    sync_all()
    t_host0 = time.perf_counter()
    evs[0].record()
    for r in range(reps):
        for _ in range(runs):
            wl.run()
        evs[r + 1].record()
    sync_all()
    t_host1 = time.perf_counter()
    ms = torch.tensor([evs[r].elapsed_time(evs[r + 1]) for r in range(reps)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = ms.tolist()
    return {"ms_per_step": statistics.median(ms) / k, "ms_per_step_sustained": sum(ms) / (reps * k),
            "ms_per_step_best": min(ms) / k, "reps": reps, "steps_per_rep": k, "region_s": sum(ms) * 1e-3,
            "host_window": (t_host0, t_host1)}


class LaunchTimer:
    """CUDA events around every fused-GEMM launch (MixedQLinear.launch_hook), on the launching stream."""

    def __init__(self):
        self.on = False
        self.records = []

    def hook(self, mod, begin):
        if not self.on:
            return
        if begin:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self.records.append([mod, e, None])
        else:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self.records[-1][2] = e

    def collect(self):
        per = {}
        for mod, a, b in self.records:
            per.setdefault(id(mod), (mod, []))[1].append(a.elapsed_time(b))
        self.records = []
        return per


def _hold_queue(ms):
    """Keeps the stream busy for about `ms` milliseconds (a spinning kernel) so that launches enqueued meanwhile run
    back to back afterwards: events around a launch then measure device time, not the host's launch rate."""
    torch.cuda._sleep(int(ms * 1.9e6))


def per_launch_roofline(wl, timer, seconds, sync_all, ms_step, world, dev):
    """The steps launched eagerly with events around each launch of the layer kernel, for about `seconds`.  The
    launches of a batch are enqueued behind a spinning kernel, so they start back to back whatever the host's speed.
    Every rank runs the same number of steps (the counts derive from figures agreed on by all ranks): the steps of a
    tensor-parallel run contain barriers among the ranks."""
    import torch.distributed as dist
    wl.reset()
    sync_all()
    t0 = time.perf_counter()
    for _ in range(3):
        wl.step()
    torch.cuda.synchronize()
    host = torch.tensor([(time.perf_counter() - t0) / 3], device=dev)
    if world > 1:
        dist.all_reduce(host, op=dist.ReduceOp.MAX)
    host_per_step = host.item()
    sync_all()
    batch = max(1, min(50, int(0.02 / max(host_per_step, 1e-5))))        # steps the host enqueues in ~20 ms
    batches = max(1, min(40, math.ceil(seconds / max(batch * ms_step * 1e-3, 1e-6))))
    timer.on = True
    for _ in range(batches):
        _hold_queue(1.3 * batch * host_per_step * 1e3 + 1.0)
        for _ in range(batch):
            wl.step()
        torch.cuda.synchronize()
    sync_all()
    timer.on = False
    return timer.collect(), batch * batches


def quantizer_times(wl, iters=30):
    """Activation-quantizer launches of the step's layers, CUDA events around each (the layers in turn, so the
    inputs of one layer have left L2 before its next launch when the step's activations exceed it); enqueued behind
    a spinning kernel so that the events see device time only."""
    from quik_b200 import asymmetric
    mods = [c.module for c in wl.cases]
    res = {}
    evs = {i: [] for i in range(len(mods))}
    ids = [m._idx16() for m in mods]
    for i, (c, m) in enumerate(zip(wl.cases, mods)):
        asymmetric.quantize_u16(c.x, ids[i][0], ids[i][1], m.bits, True)
    torch.cuda.synchronize()
    _hold_queue(25.0)
    for it in range(iters):
        for i, (c, m) in enumerate(zip(wl.cases, mods)):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            asymmetric.quantize_u16(c.x, ids[i][0], ids[i][1], m.bits, True)
            b.record()
            evs[i].append((a, b))
    torch.cuda.synchronize()
    total_bytes, total_ms = 0.0, 0.0
    for i, (c, m) in enumerate(zip(wl.cases, mods)):
        ms = statistics.fmean([a.elapsed_time(b) for a, b in evs[i]])
        nbytes = c.M * c.K * 2 + c.M * (c.K - c.F) + c.M * c.F * 2 + c.M * 4     # X in; codes (one per byte), outliers, meta out
        res[c.name] = {"us": ms * 1e3, "bytes": nbytes, "gbs": nbytes / (ms * 1e-3) / 1e9}
        total_bytes += nbytes
        total_ms += ms
    return res, total_bytes, total_ms


def gemm_plan(lib, c):
    a, b = ctypes.c_int(), ctypes.c_int()
    if lib.quik_gemm_plan(c.M, c.N, c.K - c.F, c.F, ctypes.byref(a), ctypes.byref(b)) != 0:
        return None
    return f"{'pair 256' if a.value == 2 else '128'}x{b.value}"


def measure_workload(args, wl, peaks, i8peaks, rank, world, dev, sync_all, sampler=None, want_e2e=True,
                     min_seconds=None):
    """Timed region, per-launch roofline, quantizer roofline and (optionally) e2e of one workload."""
    import torch.distributed as dist
    from quik_b200 import _lib
    from quik_b200.qlinear import MixedQLinear
    M = wl.M
    min_seconds = args.min_seconds if min_seconds is None else min_seconds
    timer = LaunchTimer()
    MixedQLinear.launch_hook = timer.hook
    for _ in range(max(args.warmup, 3)):
        wl.step()
    sync_all()
    assert _lib.device_status() == 0, "a bounded device wait ran out during warm-up"
    if not args.no_graph:
        wl.capture(sync_all, rank)
    region = timed_region(wl, args.steps, min_seconds, sync_all, world, dev)
    ms_step = region["ms_per_step"]
    value = wl.total_ops / (ms_step * 1e-3) / 1e12
    per, eager_steps = per_launch_roofline(wl, timer, min(0.5, min_seconds), sync_all, ms_step, world, dev)
    MixedQLinear.launch_hook = None

    lib = _lib.load()
    gemm_ms, gemm_ops, per_layer = 0.0, 0.0, {}
    for c in wl.cases:
        if id(c.module) not in per:
            continue
        ts = per[id(c.module)][1]
        med = statistics.fmean(ts)                         # event timestamps tick in ~2 us steps: the mean resolves finer than the median
        ops = 2.0 * M * c.N * c.K                          # this rank's shard
        gemm_ms += med
        gemm_ops += ops
        per_layer[c.name] = {"us": med * 1e3, "tops": ops / (med * 1e-3) / 1e12, "tile": gemm_plan(lib, c),
                             "shape": f"{c.K}->{c.N} int{c.bits}"}
    tensor_bound = M > 128
    achieved = gemm_ops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    peak, peak_src = i8peaks["sustained"]
    traffic = None
    if world == 1:
        t = [NCU_TRAFFIC_BYTES.get((M, c.K, c.N)) for c in wl.cases]
        if t and all(v is not None for v in t):
            traffic = sum(t) / len(t)
    kernel_alg_bytes = sum(c.M * (c.K - c.F) + c.N * (c.K - c.F) + 2 * c.F * (c.M + c.N) + 2 * c.M * c.N
                           for c in wl.cases) / len(wl.cases)
    traffic_source = NCU_TRAFFIC_SOURCE if traffic else None
    if traffic is None and world == 1 and M == 4096 and all(c.K >= 8192 for c in wl.cases):
        traffic = NCU_TRAFFIC_RATIO_70B * kernel_alg_bytes
        traffic_source = NCU_TRAFFIC_RATIO_SOURCE
    if tensor_bound:
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                    "frac": achieved / peak if peak else None, "traffic": traffic,
                    "traffic_source": traffic_source,
                    "algorithmic_bytes_per_launch": kernel_alg_bytes,
                    "kernel": "gemm_tcgen05_kernel (fused int8 GEMM + fp16 outlier GEMM + dequantize)",
                    "peak_source": f"sustained figure (the launches are timed inside a long region): {peak_src}; "
                                   f"nominal dense int8 is 4500",
                    "frac_of_burst_peak": achieved / i8peaks["burst"][0],
                    "frac_of_nominal_4500": achieved / 4500.0,
                    "per_layer": per_layer,
                    "timing": f"CUDA events around each launch of the kernel over {eager_steps} eagerly launched steps "
                              f"right after the graph-replayed region; mean per layer"}
    else:
        # few tokens: the layer is bound by reading its weights once; algorithmic bytes of the launch over its duration
        wbytes = {c.name: c.N * (c.K - c.F) * c.bits / 8 + c.N * c.F * 2 + 4 * c.N + c.M * (c.K - c.F) + 2 * c.M * c.F
                  + 2 * c.M * c.N for c in wl.cases}
        for c in wl.cases:
            if c.name in per_layer:
                per_layer[c.name]["gbs"] = wbytes[c.name] / (per_layer[c.name]["us"] * 1e-6) / 1e9
                per_layer[c.name]["hbm_frac"] = per_layer[c.name]["gbs"] / peaks["hbm_gbs"]
        tot_b = sum(wbytes[c.name] for c in wl.cases if c.name in per_layer)
        ach = tot_b / (gemm_ms * 1e-3) / 1e9 if gemm_ms > 0 else 0.0
        roofline = {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": ach / peaks["hbm_gbs"], "traffic": None,
                    "algorithmic_bytes_per_launch": tot_b / max(1, len(per_layer)),
                    "kernel": "weight-streaming layer kernels (small_m_kernel / stream_w_mma_kernel / stream_w_kernel)",
                    "peak_source": f"HBM copy bandwidth of {peaks['source']}",
                    "per_layer": per_layer,
                    "whole_step_frac": (wl.alg_bytes / (ms_step * 1e-3) / 1e9) / peaks["hbm_gbs"],
                    "whole_step_note": f"graph replay over {len(wl.sets)} rotating weight sets "
                                       f"({len(wl.sets) * sum(wbytes.values()) / 1e6:.0f} MB, L2 is {L2_BYTES / 1e6:.0f} MB); "
                                       f"algorithmic bytes of the step (weights, X, outputs) / step time, quantizers included",
                    "timing": f"CUDA events around each launch over {eager_steps} eagerly launched steps, mean per layer"}

    q_roof = None
    if world == 1:
        qres, qbytes, qms = quantizer_times(wl)
        q_roof = {"bound": "hbm", "achieved": qbytes / (qms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                  "frac": (qbytes / (qms * 1e-3) / 1e9) / peaks["hbm_gbs"], "kernel": "asym_quantize_row_kernel",
                  "per_layer": qres, "us_per_step": qms * 1e3,
                  "timing": "CUDA events around each launch, the step's layers in turn, mean of 30"}

    e2e = None
    if want_e2e and not args.no_e2e:
        e2e = measure_e2e(args, wl, rank, world, dev, sync_all)
    assert _lib.device_status() == 0, "a bounded device wait ran out"
    rec = {"value": value, "ms_per_step": ms_step, "ms_per_step_sustained": region["ms_per_step_sustained"],
           "ms_per_step_best": region["ms_per_step_best"], "timed_reps": region["reps"],
           "steps_per_rep": region["steps_per_rep"], "timed_region_s": region["region_s"], "roofline": roofline,
           "roofline_quantizer": q_roof, "e2e": e2e,
           "launch_mode": "cuda graph replay" if wl.graph is not None else "eager",
           "gpu_launches_per_step": 2 * len(wl.cases),
           "frac_of_int8_peak_whole_step": value / (peak * world) if tensor_bound else None,
           "hbm_frac_whole_step": (wl.alg_bytes / (ms_step * 1e-3) / 1e9) / peaks["hbm_gbs"]}
    if sampler is not None:
        rec["host_window"] = region["host_window"]
    return rec


def measure_e2e(args, wl, rank, world, dev, sync_all):
    """End to end through MixedQLinear.forward with host buffers.  Host side of a serving loop: uploads, layers and
    downloads run on three streams, chained per layer by events, so the two PCIe directions and the kernels overlap
    (every step still uploads all its inputs and downloads all its outputs inside the timed region).  Tensor parallel:
    every rank uploads the (replicated) activations; the assembled result is read back once, by rank 0."""
    import torch.distributed as dist
    cases, layers, M = wl.cases, wl.layers, wl.M
    wl.reset()
    dt = cases[0].x.dtype
    hx = [c.x.cpu().pin_memory() for c in cases]
    dx = [torch.empty_like(c.x) for c in cases]
    n_out = [(c.N * (world if world > 1 else 1)) for c in cases]
    ho = [torch.empty((1, M, n), dtype=dt).pin_memory() for n in n_out]
    h2d = sum(t.numel() * t.element_size() for t in hx)
    d2h = sum(t.numel() * t.element_size() for t in ho)
    if world > 1:
        h2d *= world
    s_comp = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    dout = [torch.empty((M, c.N), dtype=dt, device=dev) for c in cases] if world == 1 else None
    ev_in = [torch.cuda.Event() for _ in cases]
    ev_done = [torch.cuda.Event() for _ in cases]
    ev_out = [torch.cuda.Event() for _ in cases]
    for i, layer in enumerate(layers):
        if world == 1:
            layer.out_buffer = dout[i]
        ev_done[i].record(s_comp)
        ev_out[i].record(s_out)

    def e2e_step():
        for i, layer in enumerate(layers):
            s_in.wait_event(ev_done[i])            # the layer's previous input has been consumed
            with torch.cuda.stream(s_in):
                dx[i].copy_(hx[i], non_blocking=True)
                ev_in[i].record(s_in)
            s_comp.wait_event(ev_in[i])
            s_comp.wait_event(ev_out[i])           # the layer's previous output has been downloaded
            out = layer(dx[i].unsqueeze(0))
            if world > 1:
                layer.wait()                       # the peers' column ranges have arrived
            ev_done[i].record(s_comp)
            if rank == 0:
                s_out.wait_event(ev_done[i])
                with torch.cuda.stream(s_out):
                    ho[i].copy_(out, non_blocking=True)
                    ev_out[i].record(s_out)

    e_steps = max(3, min(args.steps, 10))
    for _ in range(3):
        e2e_step()
    sync_all()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(e_steps):
        e2e_step()
    torch.cuda.current_stream().wait_stream(s_out)         # the last download is inside the timed region
    b.record()
    sync_all()
    if world == 1:
        for layer in layers:
            layer.out_buffer = None
    ms = a.elapsed_time(b)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    return {"value": wl.total_ops / (ms / e_steps * 1e-3) / 1e12, "unit": "TOPS", "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h, "ms_per_step": ms / e_steps, "steps": e_steps}


def tp_parity(wl, shapes, M, dev, dtype, rank):
    """N > 1, outside the timed region: the assembled output of one layer on rank 0 against the un-sharded layer computed
    locally on the same seeded inputs (bit for bit: every output column is computed alike wherever it is)."""
    from quik_b200 import workloads
    idx = min(range(len(shapes)), key=lambda i: shapes[i][1] * shapes[i][2])     # the smallest layer
    name, K, N, bits = shapes[idx]
    wl.reset()
    out = wl.layers[idx](wl.cases[idx].x.unsqueeze(0))
    wl.layers[idx].wait()
    torch.cuda.synchronize()
    ok = None
    if rank == 0:
        full = workloads.make_layer(name, M, K, N, bits, seed=0, device=dev, dtype=dtype)
        want = full.module(full.x.unsqueeze(0))
        torch.cuda.synchronize()
        ok = bool(torch.equal(out, want))
        del full, want
        torch.cuda.empty_cache()
    return ok, name


def step_breakdown(wl, replays=200):
    """Where a short step's time goes: the step's layer kernels alone (token codes quantized once and reused) and its
    quantizer launches alone, each replayed from its own CUDA graph over all weight sets; microseconds per step."""
    from quik_b200 import asymmetric

    def timed(fn, steps):
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(replays):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1e3 / (replays * steps)

    mods = [[getattr(layer, "local", layer) for layer in layers] for layers in wl.sets]
    xs = [c.x for c in wl.cases]
    saved = [[m.shared_input for m in ms] for ms in mods]
    from quik_b200.qlinear import SharedQuantizedInput
    try:
        for ms in mods:
            for m in ms:
                m.shared_input = SharedQuantizedInput(1 << 60)        # quantized on the first call, then reused
        layers_only = timed(lambda: [[m(x.unsqueeze(0)) for m, x in zip(ms, xs)] for ms in mods], len(mods))
    finally:
        for ms, sv in zip(mods, saved):
            for m, sh in zip(ms, sv):
                m.shared_input = sh
    ids = [[m._idx16() for m in ms] for ms in mods]
    wide = [[not m._operand_layouts(x.shape[0])[0] for m, x in zip(ms, xs)] for ms in mods]
    quant_only = timed(lambda: [[asymmetric.quantize_u16(x, i[0], i[1], m.bits, w) for m, x, i, w in zip(ms, xs, ii, ww)]
                                for ms, ii, ww in zip(mods, ids, wide)], len(mods))
    return {"layer_kernels_alone_us_per_step": layers_only, "quantizers_alone_us_per_step": quant_only}


def tp_assembly_record(wl, world, dev, sync_all, ms_step, replays=10):
    """N > 1, outside the timed region: the assembly of every layer's output alone (no layer kernels) and the column
    shards alone (no assembly), each replayed from a CUDA graph of two steps, device time, max over ranks: the rate the
    peer copies reach against the link, the link's lower bound for a step, and the pace of the kernels by themselves."""
    import torch.distributed as dist
    if not all(hasattr(layer, "assemble_again") and layer.mode == "pull" for layer in wl.layers):
        return None

    def graph_time(fn):
        wl.reset()
        torch.cuda.synchronize()
        sync_all()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(2):
                fn()
        for _ in range(2):
            g.replay()
        torch.cuda.synchronize()
        sync_all()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(replays):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / (2 * replays)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sync_all()
        del g
        return t.item()

    for c, layer in zip(wl.cases, wl.layers):           # two forwards: both result buffers exist and hold a result
        for _ in range(2):
            layer(c.x.unsqueeze(0))
            layer.wait()
    torch.cuda.synchronize()
    pulled = [0]

    def assemble_all():
        pulled[0] = sum(layer.assemble_again() for layer in wl.layers)
        for layer in wl.layers:
            layer.wait()

    def shards_only():
        for c, layer in zip(wl.cases, wl.layers):
            layer.local.out_buffer = None
            layer.local(c.x.unsqueeze(0))

    ms = graph_time(assemble_all)
    ms_shards = graph_time(shards_only)
    link = 770.0          # GB/s per direction per GPU, measured peer copy on this pool
    bound = pulled[0] / (link * 1e9) * 1e3
    return {"pulled_bytes_per_rank_per_step": pulled[0], "assembly_alone_ms": ms,
            "assembly_alone_gbs_per_rank": pulled[0] / (ms * 1e-3) / 1e9, "link_gbs_measured_peer_copy": link,
            "link_bound_ms_per_step": bound, "step_ms_over_link_bound": ms_step / bound,
            "column_shards_alone_ms": ms_shards,
            "row_blocks": {c.name: len(layer._row_blocks(c.M, layer.local.out_features * 2))
                           for c, layer in zip(wl.cases, wl.layers)}}


def decoder_block_record(dev):
    """BASELINE config 2: one Llama-2-7B-shaped decoder block, prefill of 2048 tokens."""
    try:
        from quik_b200.block import QuikLlamaBlock
        blk = QuikLlamaBlock(4096, 32, 11008, seed=0, device=dev)
        xb = torch.randn(1, 2048, 4096, generator=torch.Generator().manual_seed(0)).half().to(dev)
        for _ in range(3):
            blk(xb)
        torch.cuda.synchronize()
        ts = []
        for _ in range(10):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            blk(xb)
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        med = statistics.median(ts)
        block = {"workload": "one Llama-2-7B decoder block (hidden 4096, 32 heads, intermediate 11008, RMSNorm, RoPE, "
                             "SDPA), all 7 linears MixedQLinear (down int8), batch 1 x 2048 tokens",
                 "ms": med, "prefill_tokens_per_s_per_block": 2048 / (med * 1e-3), "launch_mode": "eager",
                 "fused_producers": bool(getattr(blk, "fused_producers", False))}
        try:        # the same block replayed from a CUDA graph (takes the host's launch cost out)
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                blk(xb)
                torch.cuda.synchronize()
                bg = torch.cuda.CUDAGraph()
                with torch.cuda.graph(bg, stream=side):
                    blk(xb)
                bg.replay()
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(20):
                    bg.replay()
                b.record()
                torch.cuda.synchronize()
            gms = a.elapsed_time(b) / 20
            block.update({"eager_ms": med, "ms": gms, "prefill_tokens_per_s_per_block": 2048 / (gms * 1e-3),
                          "launch_mode": "cuda graph replay"})
        except Exception as exc:  # pragma: no cover
            block["graph_error"] = str(exc)[:120]
        del blk
        torch.cuda.empty_cache()
        return block
    except Exception as exc:  # pragma: no cover
        return {"error": str(exc)[:200]}


# ---------------------------------------------------------------------------------------------
def config_rows(which):
    """(config, label, M, K, N, bits, F) of every layer the benchmark configurations name."""
    from quik_b200 import workloads
    rows = []
    if which in ("0", "all"):
        rows.append((0, "single layer", 2048, 4096, 4096, 4, 256))
    if which in ("1", "all"):
        for M in (1, 16, 128, 2048):
            for (name, K, N, bits) in workloads.LLAMA2_7B:
                rows.append((1, f"7B {name}", M, K, N, bits, 256))
    if which in ("3", "all"):
        for (name, K, N, bits) in workloads.LLAMA2_70B:
            rows.append((3, f"70B {name}", 4096, K, N, bits, 256))
    if which in ("4", "all"):
        for M in (16, 4096):
            for bits in (4, 8):
                for F in (0, 128, 256, 512, 1024):
                    rows.append((4, "sweep 8192x8192", M, 8192, 8192, bits, F))
    return rows


def run_config_table(args, dev):
    """Every layer of the chosen configurations, one by one: quantizer + fused layer through MixedQLinear.forward,
    10 warm-up and 100 timed forwards with CUDA events (the method of the reference's experiments/layer_benchmark.py:12-72
    with events instead of wall clock); few-token rows are replayed from a CUDA graph over rotating copies of the
    weights that together exceed L2."""
    import copy
    from quik_b200 import _lib, workloads
    _lib.load()
    peaks = load_peaks()
    i8 = int8_peaks(peaks, measure_library_int8(dev))
    dtype = torch.float16 if args.dtype == "fp16" else torch.bfloat16
    rows = []
    for (cfg, label, M, K, N, bits, F) in config_rows(args.config):
        c = workloads.make_layer(label, M, K, N, bits, F=F, seed=0, device=dev, dtype=dtype, clip=(cfg != 4))
        ops = 2.0 * M * N * K
        wbytes = c.algorithmic_bytes
        x = c.x.unsqueeze(0)
        if M <= 128:
            weight_bytes = N * (K - F) * bits / 8 + N * F * 2
            ncopy = int(min(48, max(2, math.ceil(3 * L2_BYTES / weight_bytes))))
            mods = [c.module] + [copy.deepcopy(c.module) for _ in range(ncopy - 1)]
            for m in mods:
                m(x)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for m in mods:
                    m(x)
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
            reps = max(3, 100 // ncopy)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(reps):
                g.replay()
            b.record()
            torch.cuda.synchronize()
            us = a.elapsed_time(b) * 1e3 / (reps * ncopy)
            how = f"graph replay over {ncopy} weight copies"
            del mods, g
        else:
            for _ in range(10):
                c.module(x)
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(100):
                c.module(x)
            b.record()
            torch.cuda.synchronize()
            us = a.elapsed_time(b) * 1e3 / 100
            how = "100 eager forwards back to back"
        tops = ops / (us * 1e-6) / 1e12
        gbs = wbytes / (us * 1e-6) / 1e9
        bound = "tensor" if M > 128 else "hbm"
        frac = tops / i8["burst"][0] if bound == "tensor" else gbs / peaks["hbm_gbs"]
        rows.append({"config": cfg, "layer": label, "M": M, "K": K, "N": N, "bits": bits, "F": F, "us": us, "tops": tops,
                     "gbs": gbs, "bound": bound, "frac": frac, "how": how})
        assert _lib.device_status() == 0
        del c
        torch.cuda.empty_cache()
    print(json.dumps({"config_table": rows, "dtype": args.dtype, "int8_peak_tops": i8["burst"][0],
                      "int8_peak_source": i8["burst"][1], "hbm_peak_gbs": peaks["hbm_gbs"],
                      "timing": "quantizer + fused layer per forward (first member of a shared-input group)"}), flush=True)
    print("| config | layer | M | K -> N | bits | F | µs | TOPS | GB/s | bound | fraction of peak |", file=sys.stderr)
    print("|---|---|---|---|---|---|---|---|---|---|---|", file=sys.stderr)
    for r in rows:
        print(f"| {r['config']} | {r['layer']} | {r['M']} | {r['K']} -> {r['N']} | {r['bits']} | {r['F']} | {r['us']:.1f} | "
              f"{r['tops']:.1f} | {r['gbs']:.0f} | {r['bound']} | {r['frac']:.3f} |", file=sys.stderr)


# ---------------------------------------------------------------------------------------------
def main():
    args = parse_args()
    from quik_b200 import workloads
    shapes = workloads.LLAMA2_7B if args.model == "7b" else workloads.LLAMA2_70B
    if args.layers:
        keep = set(args.layers.split(","))
        shapes = [s for s in shapes if s[0] in keep]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    config = {"workload": f"llama2-{args.model} linear shapes {[(s[0], s[1], s[2], 'int%d' % s[3]) for s in shapes]}, "
                          f"M={args.tokens} tokens, fp_features={workloads.FP_FEATURES}, "
                          f"weights N(0,0.02) RTN+clip per channel, activations N(0,1) with x20 outlier columns, {args.dtype}",
              "tokens": args.tokens, "parallelism": f"tp{world} (output-column shards, outputs assembled on every rank)" if world > 1 else "single GPU",
              "l2": "per-step working set (weights + activations + outputs of the four layers) exceeds the 126 MB L2"}
    if args.impl == "reference":
        run_reference_arm(args, shapes, config)
        return

    import torch.distributed as dist
    from quik_b200 import _lib
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    _lib.load()
    _lib.set_engine({"auto": _lib.ENGINE_AUTO, "tcgen05": _lib.ENGINE_TCGEN05, "mma_sync": _lib.ENGINE_MMA_SYNC}[args.engine])
    _lib.set_tile_n(args.tile_n)
    if args.l2_hint >= 0:
        _lib.check(_lib.load().quik_config_set(_lib.CFG_L2_HINT, args.l2_hint), "quik_config_set")
    if args.small_m_engine >= 0:
        _lib.check(_lib.load().quik_config_set(_lib.CFG_SMALL_M, args.small_m_engine), "quik_config_set")
    if args.stream_ring >= 0:
        _lib.check(_lib.load().quik_config_set(_lib.CFG_STREAM_RING, args.stream_ring), "quik_config_set")
    if args.stream_preload >= 0:
        _lib.check(_lib.load().quik_config_set(_lib.CFG_STREAM_PRELOAD, args.stream_preload), "quik_config_set")
    if args.config:
        run_config_table(args, dev)
        return
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"          # keeps NCCL's version banner off stdout: one JSON line only
        import datetime
        # a short limit: a rank that falls out of step must end the run in minutes, not hold the GPUs
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=150))
    dtype = torch.float16 if args.dtype == "fp16" else torch.bfloat16

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    peaks = load_peaks()
    lib_int8 = measure_library_int8(dev) if (rank == 0 and not args.no_library_peak) else None
    if world > 1:
        box = [lib_int8]
        dist.broadcast_object_list(box, src=0)
        lib_int8 = box[0]
    i8peaks = int8_peaks(peaks, lib_int8)

    M = args.tokens
    # few tokens: the weights of one set of 7B layers fit in L2, so the step walks over three sets
    copies = 3 if (M <= 128 and world == 1) else 1
    wl = Workload(shapes, M, dev, dtype, world, rank, args.tp_mode, copies=copies, tp_chunks=(args.tp_chunks or None), tp_copy=args.tp_copy)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.2)
    main_rec = measure_workload(args, wl, peaks, i8peaks, rank, world, dev, sync_all, sampler=sampler)
    clocks = sampler.stop(main_rec.pop("host_window", None)) if rank == 0 else None
    if M <= 128 and world == 1:
        try:
            main_rec["breakdown"] = dict(step_breakdown(wl), step_us=main_rec["ms_per_step"] * 1e3)
        except Exception as e:
            main_rec["breakdown"] = {"error": repr(e)[:200]}
    if clocks and clocks.get("sm_mhz"):
        clocks["ms_per_step_x_sm_mhz"] = main_rec["ms_per_step"] * clocks["sm_mhz"]

    parity = None
    if world > 1:
        ok, pname = tp_parity(wl, shapes, M, dev, dtype, rank)
        parity = {"tp_parity": ok, "tp_parity_layer": pname}
        try:
            parity["tp"] = tp_assembly_record(wl, world, dev, sync_all, main_rec["ms_per_step"])
        except Exception as e:           # the record is an explanation, not the measurement
            parity["tp"] = {"error": repr(e)[:200]}
    del wl
    torch.cuda.empty_cache()

    secondary, small_m, block, cpu_base = None, None, None, None
    if world == 1 and not args.no_secondary and not args.layers:
        sub = argparse.Namespace(**vars(args))
        if not (args.model == "7b" and M == 2048):
            wl7 = Workload(workloads.LLAMA2_7B, 2048, dev, dtype)
            secondary = measure_workload(sub, wl7, peaks, i8peaks, rank, world, dev, sync_all, want_e2e=False, min_seconds=0.5)
            secondary["workload"] = "llama2-7b linear shapes (qkv, o, gate+up int4, down int8), M=2048, fp_features=256"
            del wl7
            torch.cuda.empty_cache()
        if M > 128:
            wls = Workload(workloads.LLAMA2_7B, 16, dev, dtype, copies=3)
            small_m = measure_workload(sub, wls, peaks, i8peaks, rank, world, dev, sync_all, want_e2e=False, min_seconds=0.3)
            small_m["workload"] = "llama2-7b linear shapes, M=16 tokens, fp_features=256, three rotating weight sets"
            try:
                small_m["breakdown"] = step_breakdown(wls)
                small_m["breakdown"]["step_us"] = small_m["ms_per_step"] * 1e3
            except Exception as e:
                small_m["breakdown"] = {"error": repr(e)[:200]}
            del wls
            torch.cuda.empty_cache()
        if args.dtype == "fp16":
            block = decoder_block_record(dev)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_layers, cpu_ops = cpu_fake_quant_layers(shapes, M)
        cpu_base = cpu_fake_quant_time(cpu_layers, cpu_ops, M, 2, 1)
        cpu_base = {k: cpu_base[k] for k in ("value", "unit", "cores", "kind", "sample")}

    if rank == 0:
        line = {"metric": METRIC, "value": main_rec["value"], "unit": "TOPS", "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": main_rec["ms_per_step"], "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic", "config": config,
                "roofline": main_rec["roofline"], "roofline_quantizer": main_rec["roofline_quantizer"],
                "cpu_baseline": cpu_base, "e2e": main_rec["e2e"],
                "gpu_launches": main_rec["gpu_launches_per_step"] * args.steps, "clocks": clocks,
                "launch_mode": main_rec["launch_mode"],
                "timing": {k: main_rec[k] for k in ("ms_per_step_sustained", "ms_per_step_best", "timed_reps", "steps_per_rep",
                                                    "timed_region_s")},
                "int8_tops_measured": lib_int8, "int8_peak": {k: {"tops": v[0], "source": v[1]} for k, v in i8peaks.items()},
                "frac_of_int8_peak_whole_step": main_rec["frac_of_int8_peak_whole_step"],
                "hbm_frac_whole_step": main_rec["hbm_frac_whole_step"], "activation_dtype": args.dtype,
                "secondary_7b": secondary, "small_m": small_m, "decoder_block": block}
        if parity:
            line.update(parity)
        if main_rec.get("breakdown"):
            line["breakdown"] = main_rec["breakdown"]
        print(json.dumps(line), flush=True)
    if world > 1:
        # graphs that captured collectives and symmetric-memory barriers are released before the group goes down
        sync_all()
        import gc
        gc.collect()
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
