"""Diagnostics of the few-token layer path on the GPU: where the time of a step goes.

    python -m quik_b200.diagnostics [--model 7b|70b] [--tokens 16] [--ring 0|1|2] [--preload 0|1|2]

Prints (1) the per-CTA phases of the ring streaming engine inside a replayed CUDA graph of the step, read from the
library's diagnostic counters (``quik_debug_counters``: clock64 at kernel entry, after the wait for the predecessor,
when the first block is consumed, when the last one is, after the reduction, at the end), and (2) the start and end
of every kernel of the replayed step as CUPTI reports them (torch.profiler).  Nothing here is on the product path.
"""
from __future__ import annotations

import argparse
import ctypes

import torch

from . import _lib, workloads


def _cases(model, tokens, dev, seeds):
    shapes = workloads.LLAMA2_7B if model == "7b" else workloads.LLAMA2_70B
    return shapes, [[workloads.make_layer(n, tokens, K, N, b, seed=s, device=dev) for (n, K, N, b) in shapes] for s in seeds]


def ring_phases(model="7b", tokens=16, ghz=1.9):
    """Per-CTA phase times of stream_w_mma_kernel for every layer of the step that runs on it."""
    dev = torch.device("cuda", torch.cuda.current_device())
    lib = _lib.load()
    shapes, sets = _cases(model, tokens, dev, (1, 2, 3))          # three weight sets: more than L2 holds
    bufs = {n: torch.zeros(2048 * 16, dtype=torch.int64, device=dev) for (n, _, _, _) in shapes}

    def step(trace):
        for cases in sets:
            for c, (n, _, _, _) in zip(cases, shapes):
                on = trace and cases is sets[-1]
                lib.quik_debug_counters(ctypes.c_void_p(bufs[n].data_ptr()) if on else None)
                c.module(c.x.unsqueeze(0))
        lib.quik_debug_counters(None)

    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for _ in range(3):
            step(False)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            step(True)
        for _ in range(5):
            g.replay()
        torch.cuda.synchronize()
    names = ["entry -> wait passed", "wait -> first block", "stream", "reduction", "epilogue"]
    out = {}
    for n in bufs:
        d = bufs[n].view(-1, 16).cpu()
        d = d[d[:, 8] != 0]
        if d.numel() == 0:
            continue                                       # the layer ran on another engine
        t = d[:, :6].double()
        seg = [(t[:, i + 1] - t[:, i]) / ghz / 1e3 for i in range(5)]
        out[n] = {"ctas": int(d.shape[0]), "blocks_per_cta": float(d[:, 6].double().mean()),
                  "phases_us": {nm: (float(s.mean()), float(s.min()), float(s.max())) for nm, s in zip(names, seg)},
                  "end_spread_us": float((d[:, 8].max() - d[:, 8].min()) / 1e3)}
    return out


def kernel_timeline(model="7b", tokens=16):
    """(name, start, end) in microseconds of every kernel of one replayed step."""
    from torch.profiler import ProfilerActivity, profile
    dev = torch.device("cuda", torch.cuda.current_device())
    shapes, sets = _cases(model, tokens, dev, (1,))
    cases = sets[0]

    def step():
        for c in cases:
            c.module(c.x.unsqueeze(0))

    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            step()
        for _ in range(5):
            g.replay()
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
    evs = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
    evs.sort(key=lambda e: e.time_range.start)
    last = evs[-2 * len(cases):]
    t0 = last[0].time_range.start
    return [(e.name.split("::")[-1][:40], e.time_range.start - t0, e.time_range.end - t0) for e in last]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", choices=["7b", "70b"], default="7b")
    ap.add_argument("--tokens", type=int, default=16)
    ap.add_argument("--ring", type=int, default=-1)
    ap.add_argument("--preload", type=int, default=-1)
    args = ap.parse_args()
    lib = _lib.load()
    if args.ring >= 0:
        _lib.check(lib.quik_config_set(_lib.CFG_STREAM_RING, args.ring), "quik_config_set")
    if args.preload >= 0:
        _lib.check(lib.quik_config_set(_lib.CFG_STREAM_PRELOAD, args.preload), "quik_config_set")
    for name, rec in ring_phases(args.model, args.tokens).items():
        print(f"{name}: {rec['ctas']} CTAs x {rec['blocks_per_cta']:.1f} blocks, CTAs end within {rec['end_spread_us']:.2f} us")
        for ph, (mean, lo, hi) in rec["phases_us"].items():
            print(f"    {ph:22s} mean {mean:6.2f} us  min {lo:6.2f}  max {hi:6.2f}")
    prev_end = None
    for nm, st, en in kernel_timeline(args.model, args.tokens):
        own = en - max(st, prev_end) if prev_end is not None else en - st
        print(f"{nm:40s} start {st:7.1f} end {en:7.1f} own {own:6.1f}")
        prev_end = en if prev_end is None else max(prev_end, en)


if __name__ == "__main__":
    main()
