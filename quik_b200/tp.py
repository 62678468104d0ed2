"""Tensor-parallel column split of a MixedQLinear over the ranks of a torch.distributed group.

The layer shards naturally by output channel: rank r holds rows [r*N/g, (r+1)*N/g) of int_weight,
fp_weight, weights_scales and reduced_w; the activations are replicated and every rank runs the
(cheap) quantizer itself, so no broadcast sits on the critical path.  The only exchange is one
all-gather of the M x N/g output slabs (NCCL over NVLink); the reference has no multi-GPU path
for the layer (experiments/llama.py:295-326 only places whole layers on different GPUs).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(n_total: int, world: int, rank: int, multiple: int = 8) -> slice:
    """Contiguous, equal-sized shard of the output channels (n_total must divide evenly)."""
    if n_total % (world * multiple) != 0:
        raise ValueError(f"out_features={n_total} does not split into {world} shards that are multiples of {multiple}")
    per = n_total // world
    return slice(rank * per, (rank + 1) * per)


class ColumnParallelMixedQLinear(torch.nn.Module):
    """Wraps the local shard (a MixedQLinear over N/g output channels) and assembles the full output."""

    def __init__(self, local: torch.nn.Module, group=None, gather_output: bool = True):
        super().__init__()
        self.local = local
        self.group = group
        self.gather_output = gather_output
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1

    def forward(self, x):
        out = self.local(x)                                  # [1, M, N/g]
        if self.world == 1 or not self.gather_output:
            return out
        m, n_local = out.shape[1], out.shape[2]
        slabs = torch.empty((self.world * m, n_local), dtype=out.dtype, device=out.device)
        dist.all_gather_into_tensor(slabs, out[0].contiguous(), group=self.group)
        # [g, M, N/g] -> row-major [M, N]
        return slabs.view(self.world, m, n_local).permute(1, 0, 2).reshape(1, m, self.world * n_local)
