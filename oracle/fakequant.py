"""CPU port of the reference's torch fake-quant simulation (test / baseline infrastructure).

The reference simulates the quantized layer with plain torch ops in
``experiments/quant_sim.py``; that path runs on CPU and is the timed CPU
baseline of ``bench.py`` (``cpu_baseline`` leg and ``--impl reference``).  The
reference file itself cannot travel with this repository, so this module
restates its algorithm.  It is pinned against the reference module imported
unmodified where the fixtures were generated (``tests/golden/make_golden.py``
writes ``fakequant_*.pt``; ``tests/test_oracle_golden.py`` compares).

It is *not* the parity oracle of the CUDA kernels: the simulator forces the
quantization range to include zero and uses an integer zero point in fp32
(quant_sim.py:5-7,167-188), whereas the kernels use [row-min, row-max] with a
floating zero point in fp16 (src/asymmetric/asymmetric.cu:340-435).
"""
from __future__ import annotations

import torch


def asymmetric_fake_quantize(x, scale, zero, maxq):
    """experiments/quant_sim.py:5-7."""
    q = torch.clamp(torch.round(x / scale) + zero, 0, maxq)
    return scale * (q - zero)


def symmetric_fake_quantize(x, scale, bits):
    """experiments/quant_sim.py:9-16."""
    if bits == 16:
        return x
    lo, hi = (-8, 7) if bits == 4 else (-128, 127)
    return scale * torch.clamp(torch.round(x / scale), lo, hi)


def weight_rtn_params(w: torch.Tensor, bits: int, clip: bool = True,
                      grid: int = 100, maxshrink: float = 0.8, norm: float = 2.4) -> torch.Tensor:
    """Per-output-channel symmetric RTN scale with clipping search.

    experiments/quant_sim.py:30-126 with ``perchannel=True, sym=True, mse=clip``:
    ``scale = max|w_row| / maxq``; with clipping, the shrink factor
    ``p = 1 - i/grid`` (i < maxshrink*grid) minimising ``sum |q(w) - w|^norm``
    per row is kept.  Returns scale of shape [N, 1].
    """
    maxq = 7 if bits == 4 else 127
    x = w.flatten(1)
    tmp = torch.zeros(x.shape[0], device=x.device)
    xmin = torch.minimum(x.min(1)[0], tmp)
    xmax = torch.maximum(x.max(1)[0], tmp)
    xmax = torch.maximum(torch.abs(xmin), xmax)
    neg = xmin < 0
    if torch.any(neg):
        xmin[neg] = -xmax[neg]
    dead = (xmin == 0) & (xmax == 0)
    xmin[dead] = -1
    xmax[dead] = +1
    scale = xmax / maxq
    if clip:
        best = torch.full([x.shape[0]], float("inf"), device=x.device)
        for i in range(int(maxshrink * grid)):
            p = 1 - i / grid
            scale1 = (p * xmax) / maxq
            q = symmetric_fake_quantize(x, scale1.unsqueeze(1), bits)
            q -= x
            q.abs_()
            q.pow_(norm)
            err = torch.sum(q, 1)
            better = err < best
            if torch.any(better):
                best[better] = err[better]
                scale[better] = scale1[better]
    return scale.reshape(-1, 1)


def weight_rtn_quantize(w: torch.Tensor, scale: torch.Tensor, bits: int) -> torch.Tensor:
    """experiments/quant_sim.py:128-136 (symmetric branch): the dequantized RTN weights."""
    return symmetric_fake_quantize(w, scale, bits)


def act_find_params(x: torch.Tensor, bits: int):
    """experiments/quant_sim.py:167-188 -- per-token range forced to include 0, integer zero point."""
    maxq = torch.tensor(2 ** bits - 1)
    rows = x.reshape(-1, x.shape[-1])
    tmp = torch.zeros(rows.shape[0], device=x.device)
    xmin = torch.minimum(rows.min(1)[0], tmp)
    xmax = torch.maximum(rows.max(1)[0], tmp)
    dead = (xmin == 0) & (xmax == 0)
    xmin[dead] = -1
    xmax[dead] = +1
    scale = (xmax - xmin) / maxq
    zero = torch.round(-xmin / scale)
    shape = x.shape
    scale = scale.unsqueeze(1).repeat(1, rows.shape[-1]).reshape(shape)
    zero = zero.unsqueeze(1).repeat(1, rows.shape[-1]).reshape(shape)
    return scale, zero, maxq


class FakeQuantLinear:
    """experiments/quant_sim.py:193-257 (``ActQuantWrapper`` around a bias-free ``nn.Linear``)."""

    def __init__(self, weight_dq: torch.Tensor, act_scales: torch.Tensor, fp_features: int, bits: int):
        self.weight = weight_dq                      # [N, K], already RTN-fake-quantized on int columns
        self.bits = bits
        self.fp_features_num = fp_features
        if fp_features == 0:
            self.q_idx = torch.arange(act_scales.shape[0])
            self.fp_idx = None
        else:
            order = torch.sort(act_scales)[1]
            self.fp_idx = order[-fp_features:]
            self.q_idx = order[:-fp_features]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        dt = x.dtype
        if self.bits == 16:
            return torch.nn.functional.linear(x, self.weight).to(dt)
        if self.fp_features_num == 0:
            scale, zero, maxq = act_find_params(x, self.bits)
            xq = asymmetric_fake_quantize(x, scale, zero, maxq).to(dt)
            return torch.nn.functional.linear(xq, self.weight).to(dt)
        mixed = torch.zeros_like(x)
        qf = x[..., self.q_idx]
        ff = x[..., self.fp_idx]
        scale, zero, maxq = act_find_params(qf, self.bits)
        qf = asymmetric_fake_quantize(qf, scale, zero, maxq).to(dt)
        mixed[..., self.q_idx] = qf
        mixed[..., self.fp_idx] = ff
        return torch.nn.functional.linear(mixed, self.weight).to(dt)

    __call__ = forward
