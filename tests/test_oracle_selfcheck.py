"""The reference tests' own assertions, re-expressed on the CPU oracle, plus algebraic identities."""
import pytest
import torch

from oracle import kernel_path as kp


def test_int4_matmul_reference_assertion():
    # test/python/test_matmul.py:16-26
    g = torch.Generator().manual_seed(0)
    m, k, n = 512, 512, 32
    a = torch.randint(-8, 7, (m, k), generator=g, dtype=torch.int8)
    b = torch.randint(-8, 7, (n, k), generator=g, dtype=torch.int8)
    c_gt = (a.float() @ b.float().t()).round().to(torch.int32)
    assert torch.equal(kp.int4_matmul(kp.pack_to_i4(a), kp.pack_to_i4(b)), c_gt)
    assert torch.equal(kp.int8_matmul(a, b), c_gt)


@pytest.mark.parametrize("bits", [4, 8])
def test_find_meta_reference_assertion(bits):
    # test/python/test_quant.py:11-22 (smaller matrix)
    g = torch.Generator().manual_seed(1)
    t = torch.rand((64, 1104), generator=g).half()
    xmin, xmax = t.min(1)[0], t.max(1)[0]
    unit = torch.maximum((xmax - xmin) / ((1 << bits) - 1), torch.tensor(1e-6))
    meta = kp.find_meta(t, bits)
    assert (xmin - meta[1::2]).abs().max().item() < 5e-4
    assert (meta[::2] - unit).abs().max().item() < 5e-4


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_quantize_reference_assertion(bits, dtype):
    # test/python/test_quant.py:24-39: indexed quantize == find_meta + quantizeOld on gathered columns
    g = torch.Generator().manual_seed(2)
    rows, cols, nfp = 48, 1104, 64
    t = torch.rand((rows, cols), generator=g).to(dtype)
    fp_idx = torch.randperm(cols, generator=g)[:nfp]
    int_idx = torch.arange(cols)
    int_idx = int_idx[~torch.isin(int_idx, fp_idx)]
    int_t = t[:, int_idx].contiguous()
    meta_base = kp.find_meta(int_t, bits)
    q_base = kp.quantize_old(int_t, meta_base, bits)
    q, meta, fp_t = kp.asym_quantize(t, int_idx, fp_idx, bits)
    assert torch.equal(meta, meta_base)
    assert torch.equal(fp_t, t[:, fp_idx])
    assert torch.equal(q, q_base)


@pytest.mark.parametrize("bits", [4, 8])
def test_quantizer_identity(bits):
    # x ~= (q + 2^(b-1)) * scale + zero within half a step
    g = torch.Generator().manual_seed(3)
    x = torch.randn(32, 256, generator=g).half()
    int_idx = torch.arange(256)
    q, meta, _ = kp.asym_quantize(x, int_idx, torch.tensor([], dtype=torch.long), bits)
    codes = kp.unpack_i4(q).float() if bits == 4 else q.float()
    scale, zero = meta[0::2].float()[:, None], meta[1::2].float()[:, None]
    rec = (codes + (1 << (bits - 1))) * scale + zero
    # fp16 rounding of (x - zero) and of the quotient adds up to ~1 step at 8 bits (quotients up to 255
    # carry a 0.125 ulp and the difference a 2^-8 ulp); at 4 bits the quotient is exact to << 1 step
    steps = 0.51 if bits == 4 else 1.5
    assert ((rec - x.float()).abs() <= steps * scale + 1e-3).all()
    lo, hi = -(1 << (bits - 1)), (1 << (bits - 1)) - 1
    assert codes.min() >= lo and codes.max() <= hi


def test_symmetric_reference_assertions():
    # test/python/test_cuaprseLt.py:20-23,44-47
    g = torch.Generator().manual_seed(1)
    n, k, m = 64, 256, 32
    src = torch.randn(n, k, generator=g).half()
    scale = torch.randn(n, 1, generator=g).half()
    qb = kp.sym_quantize(src, scale, 8)
    assert torch.equal(qb, (src / scale).round().to(torch.int8))
    c = torch.randn(m, n, generator=g).half()
    sr = torch.randn(m, 1, generator=g).half()
    sc = torch.randn(1, n, generator=g).half()
    y = torch.randn(m, n, generator=g).half()
    assert torch.equal(kp.sym_dequantize(c, sr, sc, y, 16), c * sr * sc + y)


def test_fused_reference_assertions():
    # test/python/test_fused.py:16-67: formulas in fp16 torch ops on small-magnitude data
    g = torch.Generator().manual_seed(2)
    m, n, k = 64, 80, 256
    a = torch.randint(-3, 3, (m, k), generator=g, dtype=torch.int8)
    b = torch.randint(-3, 3, (n, k), generator=g, dtype=torch.int8)
    sr = torch.rand(m, 1, generator=g).half()
    sc = torch.rand(1, n, generator=g).half()
    zr = torch.rand(m, 1, generator=g).half()
    wr = torch.rand(1, n, generator=g).half()
    y = torch.rand(m, n, generator=g).half()
    sv = 0.37
    c_ref = (a.float() @ b.float().t()).round().to(torch.int32)
    acc = kp.int4_matmul(kp.pack_to_i4(a), kp.pack_to_i4(b))
    assert torch.equal(acc, c_ref)
    ref_sym = c_ref * sr * sc + y
    assert torch.equal(kp.sym_fused_dequantize_fp16(acc, sr, sc, y), ref_sym)
    ref_asym = c_ref * sc * sr + (zr + torch.tensor([sv], dtype=torch.float16).item() * sr) * wr + y
    assert torch.equal(kp.asym_fused_dequantize_fp16(acc, sr, sc, sv, zr, wr, y), ref_asym)


@pytest.mark.parametrize("bits", [4, 8])
def test_layer_matches_dense_fp32_of_dequantized_operands(bits):
    """The dequant identity: the quantized path equals a dense product of the dequantized operands."""
    g = torch.Generator().manual_seed(5)
    m, k, n, nfp = 24, 192, 40, 16
    x = torch.randn(m, k, generator=g)
    fp_idx = torch.randperm(k, generator=g)[:nfp]
    x[:, fp_idx] *= 20
    x = x.half()
    w = (0.02 * torch.randn(n, k, generator=g)).half()
    maxq = 7 if bits == 4 else 127
    int_idx = torch.arange(k)
    int_idx = int_idx[~torch.isin(int_idx, fp_idx)]
    scales = w[:, int_idx].float().abs().max(dim=1, keepdim=True)[0] / maxq
    wq = (w[:, int_idx].float() / scales).round().clamp(-maxq - 1, maxq) * scales
    w_rtn = w.clone()
    w_rtn[:, int_idx] = wq.half()
    buf = kp.from_float_buffers(w_rtn, scales, fp_idx, bits)
    out = kp.mixed_linear_forward(x, buf, bits)
    # dense reference with dequantized activations and the stored (half-rounded) weight scales
    q, meta, fp_x = kp.asym_quantize(x, buf["int_indices"], buf["fp_indices"], bits)
    codes = kp.unpack_i4(q).float() if bits == 4 else q.float()
    x_dq = (codes + (1 << (bits - 1))) * meta[0::2].float()[:, None] + meta[1::2].float()[:, None]
    w_int = kp.unpack_i4(buf["int_weight"]).float() if bits == 4 else buf["int_weight"].float()
    dense = x_dq @ (w_int * buf["weights_scales"].float()).t() + fp_x.float() @ buf["fp_weight"].float().t()
    rms = dense.pow(2).mean().sqrt()
    assert (out.float() - dense).abs().max() / rms < 2e-2
