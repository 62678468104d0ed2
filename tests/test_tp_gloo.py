"""CPU, world_size 2 (gloo): host logic of the output-column tensor-parallel split."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from quik_b200.tp import ColumnParallelMixedQLinear, shard_range


def test_shard_range():
    assert shard_range(4096, 2, 1) == slice(2048, 4096)
    assert shard_range(57344, 8, 7) == slice(50176, 57344)
    with pytest.raises(ValueError):
        shard_range(100, 8, 0)


class _LocalSlab(torch.nn.Module):
    """Stand-in for the local MixedQLinear shard: x @ W[n0:n1]^T with the layer's [1, M, N/g] output shape."""

    def __init__(self, w):
        super().__init__()
        self.w = w

    def forward(self, x):
        return (x[0] @ self.w.t()).unsqueeze(0)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        m, k, n = 6, 16, 32
        x = torch.randn(1, m, k, generator=g)
        w = torch.randn(n, k, generator=g)
        sl = shard_range(n, world, rank)
        layer = ColumnParallelMixedQLinear(_LocalSlab(w[sl]))
        out = layer(x)
        ok = out.shape == (1, m, n) and torch.allclose(out[0], x[0] @ w.t(), atol=1e-6)
        local = ColumnParallelMixedQLinear(_LocalSlab(w[sl]), gather_output=False)(x)
        ok = ok and local.shape == (1, m, n // world)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_column_parallel_gather_world2():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    results = dict(q.get(timeout=10) for _ in range(2))
    assert results == {0: True, 1: True}
