"""GPU parity: activation quantizers and elementwise ops vs the CPU oracle (through the C ABI)."""
import pytest
import torch

from oracle import kernel_path as kp
from tests.gpu_util import assert_device_clean, dev, make_indices, outlier_x

pytestmark = pytest.mark.gpu

# fraction of codes allowed to differ by one step from the CPU oracle: the device division
# (__hdiv) is reciprocal based, the oracle's is IEEE; they can disagree only on quotients that
# sit within an fp32 ulp of a rounding midpoint.
CODE_MISMATCH_FRACTION = 1e-5


def _codes(q, bits, wide=False):
    if bits == 4 and not wide:
        return kp.unpack_i4(q.cpu()).to(torch.int16)
    return q.cpu().to(torch.int16)


def _check_codes(got, want, bits, wide=False):
    g, w = _codes(got, bits, wide), _codes(want, bits)
    diff = (g - w).abs()
    assert diff.max().item() <= 1
    assert (diff != 0).float().mean().item() <= CODE_MISMATCH_FRACTION, (diff != 0).sum().item()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("M,K,F,order", [
    (1, 4096, 256, "ascending"), (3, 4096, 256, "shuffled"), (17, 4096, 0, "ascending"),
    (129, 11008, 256, "ascending"), (16, 8192, 1024, "shuffled"), (5, 96, 32, "random_fp"),
    (7, 70, 4, "shuffled"), (2048, 4096, 256, "ascending"), (33, 28672, 256, "ascending"),
])
def test_asym_quantize_matches_oracle(dtype, bits, M, K, F, order):
    import quik
    ints, fp = make_indices(K, F, order)
    x = outlier_x(M, K, fp, dtype)
    q_ref, meta_ref, fp_ref = kp.asym_quantize(x, ints, fp, bits)
    xd = x.to(dev())
    q, meta, fp_x = quik.asymmetric.quantize(xd, ints.to(dev()), fp.to(dev()), bits)
    assert q.dtype == q_ref.dtype and q.shape == q_ref.shape
    assert torch.equal(meta.cpu(), meta_ref)
    assert torch.equal(fp_x.cpu(), fp_ref)
    _check_codes(q, q_ref, bits)
    # the 16-bit-id / one-code-per-byte variants must agree bit for bit with the reference layout
    from quik_b200.qlinear import _to_u16
    i16, f16 = _to_u16(ints.to(dev())), _to_u16(fp.to(dev()))
    q2, meta2, fp2 = quik.asymmetric.quantize_u16(xd, i16, f16, bits, False)
    assert torch.equal(q2, q) and torch.equal(meta2, meta) and torch.equal(fp2, fp_x)
    q3, meta3, fp3 = quik.asymmetric.quantize_u16(xd, i16, f16, bits, True)
    assert torch.equal(meta3, meta) and torch.equal(fp3, fp_x)
    assert torch.equal(_codes(q3, bits, wide=True), _codes(q, bits))
    # run twice: identical bytes (no dependence on stale shared memory)
    q4, _, _ = quik.asymmetric.quantize(xd, ints.to(dev()), fp.to(dev()), bits)
    assert torch.equal(q4, q)
    assert_device_clean()


@pytest.mark.parametrize("bits", [4, 8])
def test_reference_test_quantize(bits):
    """test/python/test_quant.py:24-39: quantize == find_meta + quantizeOld on gathered columns."""
    import quik
    torch.manual_seed(0)
    rows, cols, nfp = 512, 11088, 256
    t = torch.rand((rows, cols), dtype=torch.float16, device=dev())
    fp_indices = torch.randperm(cols)[:nfp]
    int_indices = torch.arange(cols)
    int_indices = int_indices[~torch.isin(int_indices, fp_indices)]
    fp_base = t[:, fp_indices.to(dev())]
    int_t = t[:, int_indices.to(dev())].contiguous()
    meta_base = quik.asymmetric.find_meta(int_t, bits)
    q_base = quik.asymmetric.quantizeOld(int_t, meta_base, bits)
    q, meta, fp_t = quik.asymmetric.quantize(t, int_indices.to(dev()), fp_indices.to(dev()), bits)
    assert torch.equal(meta, meta_base)
    assert torch.equal(fp_t, fp_base)
    assert torch.equal(q, q_base)
    # test_quant.py:11-22
    xmin, xmax = t.min(1)[0], t.max(1)[0]
    unit = torch.maximum((xmax - xmin) / ((1 << bits) - 1), torch.tensor(1e-6, device=dev()))
    m = quik.asymmetric.find_meta(t, bits)
    assert (xmin - m[1::2]).abs().max().item() < 5e-4
    assert (m[::2] - unit).abs().max().item() < 5e-4
    assert torch.equal(m.cpu(), kp.find_meta(t.cpu(), bits))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("rows,cols", [(1, 8), (37, 1000), (128, 4096), (5, 13)])
def test_asym_dequantize_bit_exact(dtype, bits, rows, cols):
    import quik
    g = torch.Generator().manual_seed(rows * cols + bits)
    x = torch.randint(-200000, 200000, (rows, cols), generator=g, dtype=torch.int32)
    meta = torch.stack([torch.rand(rows, generator=g) * 0.1 + 1e-3, torch.randn(rows, generator=g)], 1).reshape(-1).to(dtype)
    sc = (torch.rand(cols, 1, generator=g) * 0.01 + 1e-4).to(dtype)
    wr = torch.randn(1, cols, generator=g).to(dtype)
    y = torch.randn(rows, cols, generator=g).to(dtype)
    ref = kp.asym_dequantize(x, meta, sc, wr, y, bits)
    out = quik.asymmetric.dequantize(x.to(dev()), meta.to(dev()), sc.to(dev()), wr.to(dev()), y.to(dev()), bits)
    assert torch.equal(out.cpu(), ref)


def test_symmetric_ops_reference_assertions():
    """test/python/test_cuaprseLt.py:20-23,44-47 plus the int4 / int32 variants vs the oracle."""
    import quik
    torch.manual_seed(1)
    n, k, m = 512, 2048, 256
    src = torch.randn(n, k, dtype=torch.float16).to(dev())
    scale = torch.randn(n, 1, dtype=torch.float16).to(dev())
    qb = quik.symmetric.quantize(src, scale, 8)
    diff = (qb.cpu().to(torch.int16) - kp.sym_quantize(src.cpu(), scale.cpu(), 8).to(torch.int16)).abs()
    diff = torch.minimum(diff, 256 - diff)
    assert diff.max() <= 1 and (diff != 0).float().mean() <= 1e-5
    small = (torch.randn(n, k) * 2).half().to(dev())
    one = torch.ones(n, 1, dtype=torch.float16, device=dev())
    q4 = quik.symmetric.quantize(small, one, 4)
    assert torch.equal(q4.cpu(), kp.sym_quantize(small.cpu(), one.cpu(), 4))
    c = torch.randn(m, n, dtype=torch.float16).to(dev())
    sr = torch.randn(m, 1, dtype=torch.float16).to(dev())
    sc = torch.randn(1, n, dtype=torch.float16).to(dev())
    y = torch.randn(m, n, dtype=torch.float16).to(dev())
    assert torch.equal(quik.symmetric.dequantize(c, sr, sc, y, 16), c * sr * sc + y)
    ci = torch.randint(-2000, 2000, (m, n), dtype=torch.int32, device=dev())
    assert torch.equal(quik.symmetric.dequantize(ci, sr, sc, y, 32).cpu(),
                       kp.sym_dequantize(ci.cpu(), sr.cpu(), sc.cpu(), y.cpu(), 32))
    c8 = torch.randint(-128, 128, (m, n), dtype=torch.int8, device=dev())
    assert torch.equal(quik.symmetric.dequantize(c8, sr, sc, y, 8).cpu(),
                       kp.sym_dequantize(c8.cpu(), sr.cpu(), sc.cpu(), y.cpu(), 8))


@pytest.mark.parametrize("rows,cols", [(1, 32), (77, 96), (512, 3840)])
def test_unpack_int4(rows, cols):
    import quik
    g = torch.Generator().manual_seed(rows)
    p = torch.randint(0, 256, (rows, cols // 2), generator=g, dtype=torch.uint8)
    assert torch.equal(quik.matmul.unpack_int4(p.to(dev())).cpu(), kp.unpack_i4(p))


def test_error_paths_raise_like_the_reference():
    import quik
    x = torch.randn(4, 64, dtype=torch.float16, device=dev())
    ints, fp = make_indices(64, 8)
    with pytest.raises(RuntimeError):
        quik.asymmetric.quantize(x, ints.to(dev()), fp.to(dev()), 3)
    with pytest.raises(RuntimeError):
        quik.asymmetric.quantize(x.t(), ints.to(dev()), fp.to(dev()), 4)           # not contiguous
    with pytest.raises(RuntimeError):
        quik.asymmetric.quantize(x.cpu(), ints.to(dev()), fp.to(dev()), 4)         # not CUDA
    with pytest.raises(RuntimeError):
        quik.asymmetric.quantize(x, ints[:-2].to(dev()), fp.to(dev()), 4)          # F + K_i != K
    ints2, fp2 = make_indices(64, 7)
    with pytest.raises(RuntimeError):
        quik.asymmetric.quantize(x, ints2.to(dev()), fp2.to(dev()), 4)             # K_i odd
    with pytest.raises(RuntimeError):
        quik.matmul.int8Matmul(x, x)                                               # wrong dtype
    with pytest.raises(NotImplementedError):
        quik.matmul.int4SpMatmul(None, None, None)
