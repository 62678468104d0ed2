"""GPU parity: exact int32 GEMMs (both engines) and the fused GEMM+dequantize ops."""
import pytest
import torch

from oracle import kernel_path as kp
from quik_b200 import _lib
from tests.gpu_util import assert_device_clean, dev

pytestmark = pytest.mark.gpu

# (id, engine, tile width, CTA-pair mode: 1 = single CTAs, 2 = CTA pairs)
ENGINES = [("mma_sync", _lib.ENGINE_MMA_SYNC, 0, 0), ("auto", _lib.ENGINE_AUTO, 0, 0), ("tcgen05_auto", _lib.ENGINE_TCGEN05, 0, 0),
           ("tcgen05_1cta_n128", _lib.ENGINE_TCGEN05, 128, 1), ("tcgen05_1cta_n256", _lib.ENGINE_TCGEN05, 256, 1),
           ("tcgen05_pair_n128", _lib.ENGINE_TCGEN05, 128, 2), ("tcgen05_pair_n256", _lib.ENGINE_TCGEN05, 256, 2),
           # tile widths that are not a power of two (chosen per problem against partial waves); 240, 208, 176,
           # 144 and 48 end an epilogue warp's column range with a 16-column step
           ("tcgen05_pair_n240", _lib.ENGINE_TCGEN05, 240, 2), ("tcgen05_pair_n224", _lib.ENGINE_TCGEN05, 224, 2),
           ("tcgen05_pair_n208", _lib.ENGINE_TCGEN05, 208, 2), ("tcgen05_1cta_n176", _lib.ENGINE_TCGEN05, 176, 1),
           ("tcgen05_pair_n144", _lib.ENGINE_TCGEN05, 144, 2), ("tcgen05_1cta_n96", _lib.ENGINE_TCGEN05, 96, 1),
           ("tcgen05_pair_n48", _lib.ENGINE_TCGEN05, 48, 2),
           # the engine that moves the token operand into tensor memory (4-bit codes widened on chip): widths up to 224
           ("tcgen05_ts_auto", _lib.ENGINE_TCGEN05_TS, 0, 0), ("tcgen05_ts_pair_n224", _lib.ENGINE_TCGEN05_TS, 224, 2),
           ("tcgen05_ts_pair_n208", _lib.ENGINE_TCGEN05_TS, 208, 2), ("tcgen05_ts_pair_n192", _lib.ENGINE_TCGEN05_TS, 192, 2),
           ("tcgen05_ts_1cta_n224", _lib.ENGINE_TCGEN05_TS, 224, 1), ("tcgen05_ts_1cta_n144", _lib.ENGINE_TCGEN05_TS, 144, 1),
           ("tcgen05_ts_pair_n128", _lib.ENGINE_TCGEN05_TS, 128, 2), ("tcgen05_ts_pair_n48", _lib.ENGINE_TCGEN05_TS, 48, 2)]


@pytest.fixture(params=ENGINES, ids=[e[0] for e in ENGINES])
def engine(request):
    _, eng, tile, pair = request.param
    _lib.set_engine(eng)
    _lib.set_tile_n(tile)
    _lib.set_cta_pair(pair)
    yield request.param[0]
    torch.cuda.synchronize()
    assert_device_clean()
    _lib.set_engine(_lib.ENGINE_AUTO)
    _lib.set_tile_n(0)
    _lib.set_cta_pair(0)


SHAPES = [(128, 256, 128), (1, 8, 16), (3, 20, 48), (129, 260, 3840), (512, 32, 512), (300, 520, 10752),
          (2048, 4096, 4096), (17, 4100, 176)]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_int8_matmul_exact(engine, M, N, K):
    import quik
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randint(-128, 128, (M, K), generator=g, dtype=torch.int8)
    b = torch.randint(-128, 128, (N, K), generator=g, dtype=torch.int8)
    c = quik.matmul.int8Matmul(a.to(dev()), b.to(dev()))
    ref = kp.int8_matmul(a, b)
    assert torch.equal(c.cpu(), ref)
    c2 = quik.matmul.int8Matmul(a.to(dev()), b.to(dev()))
    assert torch.equal(c2, c)


POISON = 0x5A5A5A5A


@pytest.mark.parametrize("M,N,K", [(129, 260, 256), (300, 520, 1024), (17, 4100, 176), (256, 512, 512), (1, 8, 16)])
def test_int8_matmul_writes_only_its_output(engine, M, N, K):
    """The int32 result sits in the middle of a poisoned slab (16 rows before and after, called through the C ABI
    with a pointer into the slab): every element of [M, N] is written and nothing around it is touched.  Stands in
    for a memory checker on the ragged-edge stores of the tiled kernels."""
    from quik_b200._lib import check, load, ptr
    g = torch.Generator().manual_seed(M * 7 + N)
    a = torch.randint(-128, 128, (M, K), generator=g, dtype=torch.int8)
    b = torch.randint(-128, 128, (N, K), generator=g, dtype=torch.int8)
    pad = 16
    slab = torch.full((M + 2 * pad, N), POISON, dtype=torch.int32, device=dev())
    c = slab[pad:pad + M]
    ad, bd = a.to(dev()), b.to(dev())
    check(load().quik_int8_matmul(ptr(ad), ptr(bd), c.data_ptr(), M, N, K, torch.cuda.current_stream().cuda_stream),
          "quik_int8_matmul")
    torch.cuda.synchronize()
    assert torch.equal(c.cpu(), kp.int8_matmul(a, b))
    assert bool((slab[:pad] == POISON).all()) and bool((slab[pad + M:] == POISON).all())


@pytest.mark.parametrize("issuers", [1, 2])
@pytest.mark.parametrize("tile,pair", [(0, 0), (256, 2), (256, 1), (240, 2), (128, 1)])
@pytest.mark.parametrize("M,N,K", [(2048, 1024, 4096), (300, 520, 10752), (257, 264, 2048), (129, 4100, 28672)])
def test_two_issuing_threads_give_the_exact_product(M, N, K, tile, pair, issuers):
    """Long sums (K >= 2048) are issued by two threads that accumulate into one tensor-memory accumulator; the int32
    result must still be the exact product (any lost or torn update would show), identical to one issuing thread's,
    run after run.  Extreme codes (-128 / 127 mixed in) make every partial sum matter."""
    import quik
    g = torch.Generator().manual_seed(M + N + K + tile)
    a = torch.randint(-128, 128, (M, K), generator=g, dtype=torch.int8)
    b = torch.randint(-128, 128, (N, K), generator=g, dtype=torch.int8)
    ref = kp.int8_matmul(a, b)
    ad, bd = a.to(dev()), b.to(dev())
    try:
        _lib.set_engine(_lib.ENGINE_TCGEN05)
        _lib.set_tile_n(tile)
        _lib.set_cta_pair(pair)
        _lib.set_mma_issuers(issuers)
        for _ in range(3):
            assert torch.equal(quik.matmul.int8Matmul(ad, bd).cpu(), ref)
    finally:
        _lib.set_engine(_lib.ENGINE_AUTO)
        _lib.set_tile_n(0)
        _lib.set_cta_pair(0)
        _lib.set_mma_issuers(1)
    assert_device_clean()


@pytest.mark.parametrize("M,N,K", [(512, 32, 512), (64, 136, 3840), (2048, 512, 4096), (5, 24, 64)])
def test_int4_matmul_exact(engine, M, N, K):
    """test/python/test_matmul.py:16-26 (first shape) and ragged / Llama-sized variants."""
    import quik
    g = torch.Generator().manual_seed(K)
    a = torch.randint(-8, 8, (M, K), generator=g, dtype=torch.int8)
    b = torch.randint(-8, 8, (N, K), generator=g, dtype=torch.int8)
    c_gt = (a.float() @ b.float().t()).round().to(torch.int32)
    c = quik.matmul.int4Matmul(kp.pack_to_i4(a).to(dev()), kp.pack_to_i4(b).to(dev()))
    assert torch.equal(c.cpu(), c_gt)


def _assert_same_rounding(got, want):
    """Equal up to the rare fp16 tie that the float64 emulation of an fp32 multiply-add breaks the other way."""
    diff = (got.float() - want.float()).abs()
    ulp = torch.maximum(want.float().abs() * 2 ** -10, torch.tensor(2.0 ** -24))
    assert (diff <= ulp).all()
    assert (diff != 0).float().mean().item() < 1e-4


def _fused_inputs(bits, M, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    lo, hi = (-3, 3)
    a = torch.randint(lo, hi, (M, K), generator=g, dtype=torch.int8)
    b = torch.randint(lo, hi, (N, K), generator=g, dtype=torch.int8)
    sr = torch.rand(M, 1, generator=g).half()
    sc = torch.rand(1, N, generator=g).half()
    zr = torch.rand(M, 1, generator=g).half()
    wr = torch.rand(1, N, generator=g).half()
    y = torch.rand(M, N, generator=g).half()
    return a, b, sr, sc, zr, wr, y


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("M,N,K", [(1024, 5120, 2048), (100, 72, 256)])
def test_fused_dequantize_ops(engine, bits, M, N, K):
    """test/python/test_fused.py:16-67,130-177.  The reference asserts equality with a formula whose
    every operation is rounded to fp16; this implementation evaluates it in fp32 (fused multiply-adds)
    with one final rounding, so it must equal that fp32 formula and stay within 3 fp16 ulps of the
    largest term of the reference formula (the reference's per-op roundings scale with the terms)."""
    import quik
    a, b, sr, sc, zr, wr, y = _fused_inputs(bits, M, N, K, seed=2)
    sv = 0.4376
    acc = kp.int8_matmul(a, b)
    qa, qb = (kp.pack_to_i4(a), kp.pack_to_i4(b)) if bits == 4 else (a, b)
    d = dev()
    asym = quik.asymmetric.int4FusedDequantize if bits == 4 else quik.asymmetric.int8FusedDequantize
    sym = quik.symmetric.int4FusedDequantize if bits == 4 else quik.symmetric.int8FusedDequantize
    out = asym(qa.to(d), qb.to(d), sr.to(d), sc.to(d), sv, zr.to(d), wr.to(d), y.to(d)).cpu()
    f32 = kp.dequantize_fma(acc, sr.float(), zr.float(), sc.float(), wr.float(), y.float(), sv).half()
    _assert_same_rounding(out, f32)
    ref16 = kp.asym_fused_dequantize_fp16(acc, sr, sc, sv, zr, wr, y)
    t1 = (acc.float() * sr.float() * sc.float()).abs()
    t2 = ((zr.float() + sv * sr.float()) * wr.float()).abs()
    ulp = torch.maximum(torch.maximum(t1, t2), torch.maximum(y.float().abs(), ref16.float().abs())) * 2 ** -10
    assert ((out.float() - ref16.float()).abs() <= 3 * ulp).all()
    out_s = sym(qa.to(d), qb.to(d), sr.to(d), sc.to(d), y.to(d)).cpu()
    zero = torch.zeros_like(sr).float()
    f32s = kp.dequantize_fma(acc, sr.float(), zero, sc.float(), torch.zeros_like(sc).float(), y.float(), 0.0).half()
    _assert_same_rounding(out_s, f32s)
    ref16s = kp.sym_fused_dequantize_fp16(acc, sr, sc, y)
    ulp = torch.maximum(torch.maximum(t1, y.float().abs()), ref16s.float().abs()) * 2 ** -10
    assert ((out_s.float() - ref16s.float()).abs() <= 3 * ulp).all()
