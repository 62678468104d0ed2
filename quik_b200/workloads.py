"""Seeded synthetic workloads with the shapes and value distributions of the Llama-2 layer
benchmarks: activations ~N(0,1) with a seed-chosen set of outlier columns scaled x20, weights
~N(0, 0.02) quantized per output channel by symmetric round-to-nearest with clipping search.

These stand in for the real-model activations and checkpoints the reference's benchmarks use
(experiments/layer_benchmark.py, experiments/llama.py:328-391); no dataset or checkpoint is read.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .qlinear import MixedQLinear, SharedQuantizedInput

# (name, in_features K, out_features N, bits) -- fused-N shapes of one decoder layer
LLAMA2_7B = [("qkv", 4096, 12288, 4), ("o", 4096, 4096, 4), ("gate_up", 4096, 22016, 4), ("down", 11008, 4096, 8)]
LLAMA2_70B = [("qkv", 8192, 10240, 4), ("o", 8192, 8192, 4), ("gate_up", 8192, 57344, 4), ("down", 28672, 8192, 8)]
FP_FEATURES = 256


def rtn_clip_scales(w: torch.Tensor, bits: int, clip: bool = True, grid: int = 100, maxshrink: float = 0.8,
                    norm: float = 2.4) -> torch.Tensor:
    """Per-output-channel symmetric scale with the clipping search of the reference's weight
    quantizer (experiments/quant_sim.py:54-113 with perchannel=True, sym=True, mse=True):
    scale = p * max|w_row| / maxq for the shrink factor p = 1 - i/grid (i < maxshrink*grid) that
    minimises sum |q(w) - w|^norm.  Returns [N, 1] in w's dtype/device (computed in fp32)."""
    maxq = 7 if bits == 4 else 127
    lo, hi = (-8, 7) if bits == 4 else (-128, 127)
    x = w.float()
    xmax = x.abs().max(dim=1)[0]
    xmax = torch.where(xmax == 0, torch.ones_like(xmax), xmax)
    scale = xmax / maxq
    if clip:
        best = torch.full_like(xmax, float("inf"))
        for i in range(int(maxshrink * grid)):
            p = 1 - i / grid
            s1 = (p * xmax) / maxq
            q = s1[:, None] * torch.clamp(torch.round(x / s1[:, None]), lo, hi)
            err = (q - x).abs_().pow_(norm).sum(1)
            better = err < best
            best = torch.where(better, err, best)
            scale = torch.where(better, s1, scale)
    return scale.reshape(-1, 1)


@dataclass
class LayerCase:
    name: str
    M: int
    K: int
    N: int
    F: int
    bits: int
    x: torch.Tensor                 # [M, K] activations (device)
    module: MixedQLinear
    fp_indices: torch.Tensor        # ascending outlier column ids (cpu)
    weight_dq: torch.Tensor | None  # [N, K] fake-quantized weights (what the simulator multiplies by)

    @property
    def ops(self) -> float:
        return 2.0 * self.M * self.N * self.K

    @property
    def algorithmic_bytes(self) -> float:
        k_i = self.K - self.F
        return (self.N * k_i * self.bits / 8 + self.N * self.F * 2 + 2 * self.N * 2
                + self.M * self.K * 2 + self.M * self.N * 2)


def make_layer(name: str, M: int, K: int, N: int, bits: int, F: int = FP_FEATURES, seed: int = 0,
               device="cuda", dtype=torch.float16, n_slice: slice | None = None, keep_weight_dq: bool = False,
               shared_input: SharedQuantizedInput | None = None, clip: bool = True) -> LayerCase:
    """One layer of the benchmark: seeded X [M,K] and a MixedQLinear built by ``from_float``.

    ``n_slice`` keeps only a slice of the output channels (tensor-parallel column shard): the full
    weight matrix is generated from the seed and then sliced, so shards of different ranks are
    consistent with the single-GPU layer.
    """
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    fp_idx = torch.randperm(K, generator=g)[:F]
    if F > 0:
        x[:, fp_idx] *= 20
    w = 0.02 * torch.randn(N, K, generator=g)
    if n_slice is not None:
        w = w[n_slice].contiguous()
    x = x.to(dtype).to(device)
    w = w.to(dtype).to(device)
    # outlier ids in the order the reference derives them: ascending activation scale, here a
    # stand-in that is 1 on outlier columns and 0 elsewhere (stable sort -> ascending column id)
    standin = torch.zeros(K)
    standin[fp_idx] = 1.0
    fp_sorted = torch.sort(standin, stable=True)[1][K - F:] if F > 0 else torch.tensor([], dtype=torch.long)
    int_mask = torch.ones(K, dtype=torch.bool)
    int_mask[fp_sorted] = False
    int_cols = torch.arange(K)[int_mask].to(device)
    scales = rtn_clip_scales(w[:, int_cols], bits, clip=clip)
    lo, hi = (-8, 7) if bits == 4 else (-128, 127)
    w_rtn = w.clone()
    w_rtn[:, int_cols] = (scales * torch.clamp(torch.round(w[:, int_cols].float() / scales), lo, hi)).to(dtype)
    lin = torch.nn.Linear(K, w.shape[0], bias=False)
    mod = MixedQLinear.from_float(lin, w_rtn, scales, shared_input=shared_input,
                                  fp_indices=fp_sorted if F > 0 else None, bits=bits).to(device)
    return LayerCase(name, M, K, w.shape[0], F, bits, x, mod, fp_sorted, w_rtn if keep_weight_dq else None)


def standin_act_scales(K: int, fp_indices: torch.Tensor) -> torch.Tensor:
    s = torch.zeros(K)
    if fp_indices.numel():
        s[fp_indices] = 1.0
    return s
