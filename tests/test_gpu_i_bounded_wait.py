"""GPU: a device-side wait that cannot complete runs out, is reported, and leaves the context usable.

Every mbarrier wait of the tcgen05 kernels is bounded (two seconds in the product kernels).  The library's self-test
kernel runs the same wait routine on a barrier nothing arrives on with a limit of a few milliseconds: the kernel must
return by itself, the device status must read QUIK_ERR_DEVICE_WAIT exactly once (reading clears it), and a normal
layer launched afterwards must work.  Nothing is made to fault, trap or hang.
"""
import time

import pytest
import torch

from quik_b200 import _lib
from quik_b200.workloads import make_layer

pytestmark = pytest.mark.gpu
QUIK_ERR_DEVICE_WAIT = -9


def test_wait_that_cannot_complete_runs_out_and_is_reported():
    lib = _lib.load()
    dev = torch.device("cuda:0")
    assert _lib.device_status() == 0
    result = torch.zeros(1, dtype=torch.int32, device=dev)
    t0 = time.perf_counter()
    rc = lib.quik_selftest_bounded_wait(3000, result.data_ptr(), torch.cuda.current_stream().cuda_stream)   # 3 ms
    assert rc == 0, lib.quik_strerror(rc)
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    assert elapsed < 1.0, f"the bounded wait took {elapsed:.3f} s"
    assert int(result.item()) == 2                       # the wait gave up and raised the abort flag
    assert lib.quik_device_status(1) == QUIK_ERR_DEVICE_WAIT
    assert b"wait ran out" in lib.quik_strerror(QUIK_ERR_DEVICE_WAIT)
    assert lib.quik_device_status(1) == 0                # cleared by the read
    # the context is intact: a layer runs and reports a clean status
    case = make_layer("t", 300, 1088, 520, 4, F=64, seed=1, device=dev, clip=False)
    out = case.module(case.x.unsqueeze(0))
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    assert _lib.device_status() == 0


def test_selftest_rejects_unbounded_limits():
    lib = _lib.load()
    assert lib.quik_selftest_bounded_wait(0, None, None) != 0
    assert lib.quik_selftest_bounded_wait(2_000_000, None, None) != 0
