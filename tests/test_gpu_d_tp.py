"""GPU, 2 ranks (skipped with fewer than 2 GPUs): the tensor-parallel layer assembles the same [M, N]
output as the single-GPU layer, with both assembly paths (copy-engine pulls, NCCL all-gather)."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from quik_b200.tp import ColumnParallelMixedQLinear, shard_range
        from quik_b200.workloads import make_layer
        M, K, N = 512, 1024, 1024
        full = make_layer("f", M, K, N, 4, F=64, seed=3, device=dev, clip=False)
        want = full.module(full.x.unsqueeze(0))
        res = {}
        for key, mode, chunks in (("nccl", "nccl", None), ("pull", "pull", None), ("pull_blocks", "pull", 2),
                                  ("pull_sm", "pull", None)):
            shard = make_layer("s", M, K, N, 4, F=64, seed=3, device=dev, clip=False, n_slice=shard_range(N, world, rank))
            layer = ColumnParallelMixedQLinear(shard.module, mode=mode, chunks=chunks,      # chunks=2: two row blocks of 256
                                               copy="auto" if key == "pull_sm" else "ce")  # auto: these 1 KB rows go through the copy kernel
            ok = True
            for i in range(5):                      # repeated calls alternate between the two result buffers
                xi = (full.x * (1.0 + 0.25 * i)).contiguous()
                want_i = want if i == 0 else full.module(xi.unsqueeze(0))
                got = layer(xi.unsqueeze(0))
                if mode == "pull":
                    layer.wait()
                torch.cuda.synchronize()
                ok = ok and bool(torch.equal(got, want_i))
            if mode == "pull":
                # the same as a CUDA graph of four forwards (an even number keeps the buffer alternation across
                # replays), replayed three times without host work in between
                layer.reset()
                torch.cuda.synchronize()
                dist.barrier()
                xs = [(full.x * (1.0 + 0.5 * i)).contiguous() for i in range(4)]
                wants = [full.module(x.unsqueeze(0)).clone() for x in xs]
                g = torch.cuda.CUDAGraph()
                outs = []
                with torch.cuda.graph(g):
                    for i, x in enumerate(xs):
                        o = layer(x.unsqueeze(0))
                        if i >= 2:
                            layer.wait()
                            outs.append(o.clone())         # forwards 2 and 3 own the two buffers at the end
                    layer.wait()
                for _ in range(3):
                    g.replay()
                torch.cuda.synchronize()
                ok = ok and bool(torch.equal(outs[0], wants[2])) and bool(torch.equal(outs[1], wants[3]))
                # drop every reference to this layer's symmetric buffers now: a view that lived on into the next
                # variant's capture would free them there, which a capturing stream does not permit
                del o, g, outs
            del got, layer, shard
            torch.cuda.synchronize()
            res[key] = ok
        q.put((rank, res))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tensor_parallel_two_ranks():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    results = dict(q.get(timeout=10) for _ in range(2))
    good = {"nccl": True, "pull": True, "pull_blocks": True, "pull_sm": True}
    assert results == {0: good, 1: good}


@pytest.mark.parametrize("rows,width,ctas", [(64, 4096, 0), (333, 5120, 7), (1, 16, 1), (4096, 2048, 32)])
def test_copy_2d_on_the_sms_copies_a_column_range(rows, width, ctas):
    """quik_copy_2d_sm (the kernel form of the assembly copy) on local memory: the column range arrives, the
    bytes beside it stay untouched; misaligned widths are refused."""
    from quik_b200._lib import load
    lib = load()
    pitch_s, pitch_d = width * 3, width * 2
    src = torch.randint(0, 255, (rows, pitch_s), dtype=torch.uint8, device="cuda")
    dst = torch.full((rows, pitch_d), 7, dtype=torch.uint8, device="cuda")
    rc = lib.quik_copy_2d_sm(dst.data_ptr() + width, pitch_d, src.data_ptr() + 2 * width, pitch_s, width, rows, ctas,
                             torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(dst[:, width:], src[:, 2 * width:])
    assert bool((dst[:, :width] == 7).all())
    assert lib.quik_copy_2d_sm(dst.data_ptr(), pitch_d, src.data_ptr(), pitch_s, 24, rows, 0, None) != 0
