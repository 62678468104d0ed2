"""GPU test of the no-allocation int4 GEMM entry point (collected last on purpose).

quik_int4_matmul_fixed_scratch serves hosts that cannot call cudaMalloc when they need the product
(all device memory already handed to their own pool, or no tolerance for the synchronisation an
allocation may imply): its scratch is a fixed array inside the library instead of caller memory.
The test drives it through the C ABI, twice in a row with different operands and shapes -- the
second call finds the first call's leftovers in the shared array -- and demands the very same int32
results as the regular entry point and as the CPU oracle's exact integer product, plus a clean refusal
of sizes beyond the fixed area.  Where a second GPU is present the small case is repeated there: the
array's device address is looked up per device.
"""
import pytest
import torch

from oracle import kernel_path as kp
from quik_b200 import _lib
from quik_b200._lib import load, ptr

pytestmark = pytest.mark.gpu

NOALLOC_SCRATCH_BYTES = 16 << 20


def _both(lib, a, b):
    M, N, K = a.shape[0], b.shape[0], a.shape[1] * 2
    st = torch.cuda.current_stream().cuda_stream
    want = torch.empty((M, N), dtype=torch.int32, device=a.device)
    nbytes = lib.quik_int4_matmul_scratch_bytes(M, N, K)
    scratch = torch.empty((nbytes,), dtype=torch.uint8, device=a.device)
    rc = lib.quik_int4_matmul(ptr(a), ptr(b), ptr(want), M, N, K, ptr(scratch), nbytes, st)
    assert rc == 0, lib.quik_strerror(rc)
    got = torch.full((M, N), -7, dtype=torch.int32, device=a.device)
    rc = lib.quik_int4_matmul_fixed_scratch(ptr(a), ptr(b), ptr(got), M, N, K, st)
    assert rc == 0, lib.quik_strerror(rc)
    torch.cuda.synchronize()
    return got, want


def test_fixed_scratch_matches_regular_entry_point_twice():
    lib = load()
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(123)
    # first call: a large-ish problem that fills most of what a later, smaller call will reuse
    a1 = torch.randint(0, 256, (1024, 1920), generator=g, dtype=torch.uint8).to(dev)
    b1 = torch.randint(0, 256, (2048, 1920), generator=g, dtype=torch.uint8).to(dev)
    got1, want1 = _both(lib, a1, b1)
    assert torch.equal(got1, want1)
    # second call, straight after: different shape (ragged M and N) and values over the stale contents
    a2 = torch.randint(0, 256, (77, 256), generator=g, dtype=torch.uint8).to(dev)
    b2 = torch.randint(0, 256, (136, 256), generator=g, dtype=torch.uint8).to(dev)
    got2, want2 = _both(lib, a2, b2)
    assert torch.equal(got2, want2)
    # both against the oracle's exact integer product of the same packed operands
    assert torch.equal(got1.cpu(), kp.int4_matmul(a1.cpu(), b1.cpu()))
    assert torch.equal(got2.cpu(), kp.int4_matmul(a2.cpu(), b2.cpu()))
    # and the first problem again gives the first answer again
    got3, _ = _both(lib, a1, b1)
    assert torch.equal(got3, want1)
    assert _lib.device_status() == 0


def test_fixed_scratch_on_a_second_device():
    """The fixed array exists once per GPU; its address is looked up with that GPU current."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    lib = load()
    g = torch.Generator().manual_seed(5)
    a = torch.randint(0, 256, (77, 256), generator=g, dtype=torch.uint8)
    b = torch.randint(0, 256, (136, 256), generator=g, dtype=torch.uint8)
    want = kp.int4_matmul(a, b)
    for d in (1, 0):
        with torch.cuda.device(d):
            got, same = _both(lib, a.to(f"cuda:{d}"), b.to(f"cuda:{d}"))
            assert torch.equal(got.cpu(), want) and torch.equal(same.cpu(), want)


def test_fixed_scratch_empty_problem_is_ok_whatever_the_other_size():
    lib = load()
    rc = lib.quik_int4_matmul_fixed_scratch(None, None, None, 0, 1 << 20, 4096, torch.cuda.current_stream().cuda_stream)
    assert rc == 0


def test_fixed_scratch_rejects_sizes_beyond_its_area():
    lib = load()
    dev = torch.device("cuda:0")
    K = 4096
    M, N = 2048, 4096                      # (M + N) * K = 24 Mi > 16 Mi
    assert lib.quik_int4_matmul_scratch_bytes(M, N, K) > NOALLOC_SCRATCH_BYTES
    a = torch.zeros((M, K // 2), dtype=torch.uint8, device=dev)
    b = torch.zeros((N, K // 2), dtype=torch.uint8, device=dev)
    c = torch.full((M, N), 5, dtype=torch.int32, device=dev)
    rc = lib.quik_int4_matmul_fixed_scratch(ptr(a), ptr(b), ptr(c), M, N, K, torch.cuda.current_stream().cuda_stream)
    assert rc == -10
    assert b"fixed scratch" in lib.quik_strerror(rc)
    torch.cuda.synchronize()
    assert bool((c == 5).all())            # nothing was launched
    # the largest problem that still fits is accepted
    M2, N2 = 512, 3584                     # (M + N) * K = 16 Mi exactly
    assert lib.quik_int4_matmul_scratch_bytes(M2, N2, K) == NOALLOC_SCRATCH_BYTES
    rc = lib.quik_int4_matmul_fixed_scratch(ptr(a), ptr(b), ptr(c), M2, N2, K, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert bool((c[:M2].reshape(-1)[: M2 * N2] == 0).all())
