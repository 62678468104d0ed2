#!/usr/bin/env python
"""Benchmark of the MixedQLinear hot path on B200.

One step = one pass of the four linear layers of a Llama-2 decoder layer (fused-N shapes: qkv,
o, gate+up int4 with 256 fp16 outlier columns, down int8) over M tokens of seeded synthetic
activations: activation quantizer + fused int GEMM / outlier GEMM / dequantize per layer.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens M] [--model 7b|70b] [--impl reference]

Prints one JSON line (rank 0).  `value` is whole-job TOPS (2*M*N*K summed over the layers / time)
with inputs resident in HBM; `e2e` is the same metric through MixedQLinear.forward with the
activations copied from pinned host memory and the outputs copied back inside the timed region.
N > 1 (torchrun): the layers are column-sharded over the ranks and the outputs all-gathered.
`--impl reference` times the reference's torch fake-quant simulation of the same layers on the
host cores (a port of it; the reference checkout is not needed at run time).
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

import torch  # noqa: E402

METRIC = "MixedQLinear TOPS (Llama-2 linear shapes, fused quantize+GEMM+dequant)"
# dram__bytes_read.sum + dram__bytes_write.sum per launch of gemm_tcgen05_kernel at M = 2048, F = 256, from one
# `ncu --set full` capture of a bench step (profiles/gemm_tcgen05_llama7b_m2048.md); key = (K, N)
NCU_TRAFFIC_BYTES_M2048 = {(4096, 12288): 84.55e6, (4096, 4096): 26.88e6, (4096, 22016): 178.77e6, (11008, 4096): 84.54e6}
CPU_SAMPLE_TOKENS = 256


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--model", choices=["7b", "70b"], default="7b")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--engine", choices=["auto", "tcgen05", "mma_sync"], default="auto")
    ap.add_argument("--tile-n", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--layers", default="", help="comma-separated subset of layer names")
    ap.add_argument("--no-block", action="store_true",
                    help="skip the decoder-block prefill measurement (BASELINE config 2) that rides along at N=1")
    ap.add_argument("--no-graph", action="store_true",
                    help="time eager launches instead of replaying the step as a CUDA graph")
    ap.add_argument("--tp-mode", choices=["pull", "nccl"], default="pull",
                    help="N > 1: assemble outputs by copy-engine pulls from symmetric memory, or by NCCL all-gather")
    return ap.parse_args()


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs."""
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
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------------
def cpu_fake_quant_baseline(shapes, tokens, steps, warmup, seed=0):
    """The reference's torch fake-quant simulation (experiments/quant_sim.py ActQuantWrapper around
    nn.Linear with RTN-quantized weights), ported in oracle/fakequant.py, timed on the host cores."""
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
        layer.weight = w
        layers.append((layer, x.half()))
        ops += 2.0 * tokens * N * K
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
            "sample": f"{tokens} of the workload's tokens per layer, all {len(shapes)} layers, "
                      f"{steps} timed passes after {warmup} warm-up (oracle/fakequant.py on "
                      f"{os.cpu_count()} host cores)", "ms_per_step": mean * 1e3}


def run_reference_arm(args, shapes, config):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 20))
    warm = max(1, min(args.warmup, 3))
    base = cpu_fake_quant_baseline(shapes, CPU_SAMPLE_TOKENS, steps, warm)
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": "TOPS", "n_gpus": args.gpus,
            "steps": steps, "warmup": warm, "ms_per_step": base["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic", "config": config,
            "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": base["value"], "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


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
                          f"weights N(0,0.02) RTN+clip per channel, activations N(0,1) with x20 outlier columns",
              "tokens": args.tokens, "parallelism": f"tp{world} (output-column shards + all-gather)" if world > 1 else "single GPU",
              "l2": "per-step working set (weights + activations + outputs of the four layers) exceeds the 126 MB L2"}
    if args.impl == "reference":
        run_reference_arm(args, shapes, config)
        return

    import torch.distributed as dist
    from quik_b200 import _lib
    from quik_b200.qlinear import MixedQLinear
    from quik_b200.tp import ColumnParallelMixedQLinear, shard_range
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()
    _lib.set_engine({"auto": _lib.ENGINE_AUTO, "tcgen05": _lib.ENGINE_TCGEN05, "mma_sync": _lib.ENGINE_MMA_SYNC}[args.engine])
    _lib.set_tile_n(args.tile_n)

    M = args.tokens
    cases, layers = [], []
    for (name, K, N, bits) in shapes:
        sl = shard_range(N, world, rank) if world > 1 else None
        c = workloads.make_layer(name, M, K, N, bits, seed=0, device=dev, n_slice=sl)
        cases.append(c)
        layers.append(ColumnParallelMixedQLinear(c.module, mode=args.tp_mode) if world > 1 else c.module)
        torch.cuda.empty_cache()
    total_ops = sum(2.0 * M * N * K for (_, K, N, _) in shapes)          # whole job, all ranks
    alg_bytes = sum(c.algorithmic_bytes for c in cases)

    # ---- CUDA-event hook around the fused GEMM launch (roofline of the dominant kernel)
    pool = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            for _ in range(len(shapes) * (args.steps + 1))]
    used = []
    state = {"on": False, "i": 0}

    def hook(mod, begin):
        if not state["on"]:
            return
        if begin:
            pool[state["i"]][0].record()
        else:
            pool[state["i"]][1].record()
            used.append((state["i"], mod))
            state["i"] += 1

    MixedQLinear.launch_hook = hook

    def step():
        outs = []
        for c, layer in zip(cases, layers):
            outs.append(layer(c.x.unsqueeze(0)))
        if world > 1:
            for layer in layers:
                layer.wait()          # the assembled outputs are part of the step
        return outs

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    sync_all()
    assert _lib.device_status() == 0, "a bounded device wait ran out during warm-up"

    # ---- the step as a CUDA graph: the launches (two per layer, plus the output assembly for N > 1)
    # are replayed without host work in between; falls back to eager launches if capture fails
    graph = None
    if not args.no_graph:
        try:
            for layer in layers:
                if hasattr(layer, "reset"):
                    layer.reset()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                graph_outs = step()
            graph = g
            for _ in range(3):
                graph.replay()
            sync_all()
        except Exception as exc:  # pragma: no cover - depends on the runtime
            if rank == 0:
                print(f"# CUDA graph capture failed, timing eager launches: {exc}", file=sys.stderr)
            graph = None
            sync_all()

    def run_step():
        if graph is not None:
            graph.replay()
        else:
            step()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    e0.record()
    for _ in range(args.steps):
        run_step()
    e1.record()
    sync_all()
    ms_total = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = t.item()
    ms_step = ms_total / args.steps
    value = total_ops / (ms_step * 1e-3) / 1e12

    # ---- the same steps launched eagerly with CUDA events around every fused-GEMM launch (events
    # cannot be timed inside a replayed graph); still inside the clock-sampling window
    sync_all()
    for layer in layers:
        if hasattr(layer, "reset"):
            layer.reset()             # events recorded during capture must not be waited on eagerly
    state["on"] = True
    ee0, ee1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ee0.record()
    for _ in range(args.steps):
        step()
    ee1.record()
    sync_all()
    state["on"] = False
    eager_ms_step = ee0.elapsed_time(ee1) / args.steps
    clocks = sampler.stop() if rank == 0 else None

    # ---- dominant-kernel roofline (this rank's launches)
    gemm_ms, gemm_ops, per_layer = 0.0, 0.0, {}
    for i, mod in used:
        dt = pool[i][0].elapsed_time(pool[i][1])
        ops = 2.0 * M * mod.out_features * mod.in_features
        gemm_ms += dt
        gemm_ops += ops
        key = f"{mod.in_features}->{mod.out_features} int{mod.bits}"
        per_layer.setdefault(key, []).append(dt)
    peaks = load_peaks()
    int8_peak = 2.0 * peaks["bf16_tflops"]
    achieved = gemm_ops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    traffic = None
    if world == 1 and M == 2048 and args.model == "7b" and used:
        per = [NCU_TRAFFIC_BYTES_M2048.get((mod.in_features, mod.out_features)) for _, mod in used]
        if all(v is not None for v in per):
            traffic = sum(per) / len(per)          # bytes per launch, averaged over the timed launches
    roofline = {"bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TFLOP/s",
                "frac": achieved / int8_peak if int8_peak else None, "traffic": traffic,
                "algorithmic_bytes_per_launch": sum(c.M * (c.K - c.F) + c.N * (c.K - c.F) + 2 * c.F * (c.M + c.N)
                                                    + 2 * c.M * c.N for c in cases) / len(cases),
                "kernel": "gemm_tcgen05_kernel (fused int8 GEMM + fp16 outlier GEMM + dequantize)",
                "peak_source": f"2 x bf16 dense GEMM peak of {peaks['source']} ({peaks['bf16_tflops']} TF/s burst); "
                               f"int8 runs at twice the bf16 rate on this part; nominal dense int8 is 4500",
                "frac_of_nominal_4500": achieved / 4500.0,
                "per_layer_us": {k: 1e3 * sum(v) / len(v) for k, v in per_layer.items()},
                "timing": "CUDA events around each launch of the kernel, recorded while the timed steps are "
                          "launched eagerly right after the graph-replayed timing loop",
                "hbm_frac_whole_step": (alg_bytes / (ms_step * 1e-3) / 1e9) / peaks["hbm_gbs"]}

    # ---- end to end through the public API with host buffers
    e2e = None
    if not args.no_e2e:
        hx = [c.x.cpu().pin_memory() for c in cases]
        dx = [torch.empty_like(c.x) for c in cases]
        n_out = [(c.N * (world if world > 1 else 1)) for c in cases]
        ho = [torch.empty((1, M, n), dtype=torch.float16).pin_memory() for n in n_out]
        h2d = sum(t.numel() * t.element_size() for t in hx)
        d2h = sum(t.numel() * t.element_size() for t in ho)

        # Host side of a serving loop: uploads, layers and downloads run on three streams, chained per layer by
        # events, so the two PCIe directions and the kernels overlap (every step still uploads all its inputs and
        # downloads all its outputs inside the timed region).  Tensor parallel: every rank uploads the (replicated)
        # activations; the assembled result is read back once, by rank 0.
        if world > 1:
            h2d *= world
        s_comp = torch.cuda.current_stream()
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        dout = [torch.empty((M, c.N), dtype=torch.float16, device=dev) for c in cases] if world == 1 else None
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
        e2e = {"value": total_ops / (ms / e_steps * 1e-3) / 1e12, "unit": "TOPS", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": ms / e_steps, "steps": e_steps}
    assert _lib.device_status() == 0, "a bounded device wait ran out"

    # ---- BASELINE config 2 rides along: one Llama-2-7B-shaped decoder block, prefill of 2048 tokens
    block = None
    if world == 1 and not args.no_block and args.model == "7b" and M == 2048:
        try:
            from quik_b200.block import QuikLlamaBlock
            MixedQLinear.launch_hook = None
            del cases, layers
            torch.cuda.empty_cache()
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
                     "ms": med, "prefill_tokens_per_s_per_block": 2048 / (med * 1e-3), "launch_mode": "eager"}
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
                    for _ in range(10):
                        bg.replay()
                    b.record()
                    torch.cuda.synchronize()
                gms = a.elapsed_time(b) / 10
                block.update({"eager_ms": med, "ms": gms, "prefill_tokens_per_s_per_block": 2048 / (gms * 1e-3),
                              "launch_mode": "cuda graph replay"})
            except Exception as exc:  # pragma: no cover
                block["graph_error"] = str(exc)[:120]
        except Exception as exc:  # pragma: no cover
            block = {"error": str(exc)[:200]}

    cpu_base = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_base = cpu_fake_quant_baseline(shapes, CPU_SAMPLE_TOKENS, 5, 1)
        cpu_base = {k: cpu_base[k] for k in ("value", "unit", "cores", "kind", "sample")}

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": "TOPS", "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "int8", "data": "synthetic", "config": config, "roofline": roofline,
                "cpu_baseline": cpu_base, "e2e": e2e, "gpu_launches": 2 * len(shapes) * args.steps, "clocks": clocks,
                "launch_mode": "cuda graph replay" if graph is not None else "eager", "eager_ms_per_step": eager_ms_step,
                "decoder_block": block,
                "frac_of_int8_peak_whole_step": value / (int8_peak * world)}
        print(json.dumps(line), flush=True)
    if world > 1:
        # leave without tearing the communicators down: graph-captured collectives and symmetric-memory
        # handles make an orderly destroy slow or blocking on some runtimes, and the result is printed
        sync_all()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
