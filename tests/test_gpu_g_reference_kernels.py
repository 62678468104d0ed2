"""GPU parity against the reference's OWN CUDA kernels on the same inputs.

oracle/build_ref.py compiles the QUIK reference's CUDA sources unmodified from the reference checkout
(src/asymmetric/{asymmetric,fused_dequantize}.cu, src/symmetric/{symmetric,fused_dequantize}.cu, src/matmul/matmul.cu:
quantize, quantizeOld, find_meta, dequantize, the symmetric ops, the CUTLASS int4 / int8 GEMMs and the fused GEMM +
dequantize ops) into oracle/_ref/.  These tests run them on the GPU next to this repository's kernels, and next to the
CPU oracle, on the same inputs.  They are skipped when that library is absent (it is built where the reference
checkout is available and travels with the repository's other built files).

Shapes respect what the reference kernels assume: at least 1024 elements (its block size then is the power of two its
tree reduction needs), at least 1024 columns for the fused quantizer (one row per block: its blocks do not
synchronise between rows), power-of-two columns for find_meta, an even element count for dequantize.
"""
import pytest
import torch

from oracle import build_ref
from tests.gpu_util import assert_device_clean, dev, rel_rms_err

pytestmark = pytest.mark.gpu

_ref = None


def ref_ops():
    global _ref
    if _ref is None:
        _ref = build_ref.load() or False
    if not _ref:
        pytest.skip("oracle/_ref (reference kernels) not built")
    return _ref


def _indices(cols, nfp, order, seed):
    g = torch.Generator().manual_seed(seed)
    fp = torch.randperm(cols, generator=g)[:nfp]
    ints = torch.arange(cols)
    ints = ints[~torch.isin(ints, fp)]
    if order == "ascending":
        fp = fp.sort()[0]
    else:
        ints = ints[torch.randperm(ints.numel(), generator=g)]
    return ints, fp


def _activations(rows, cols, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g)
    x[:, torch.randperm(cols, generator=g)[: max(1, cols // 16)]] *= 20.0
    return x.to(dtype)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("rows,cols,nfp,order", [
    (16, 4352, 256, "ascending"), (129, 11264, 256, "ascending"), (2048, 4352, 256, "shuffled"),
    (7, 1024, 0, "ascending"), (33, 8192 + 1024, 1024, "shuffled"), (1, 2048, 64, "ascending"),
])
def test_asym_quantize_equals_reference_kernel(dtype, bits, rows, cols, nfp, order):
    """quik.asymmetric.quantize (asymmetric.cu:340-584): codes, meta and outlier columns, byte for byte."""
    import quik
    ref = ref_ops()
    x = _activations(rows, cols, dtype, rows + cols + bits).to(dev())
    ints, fp = _indices(cols, nfp, order, cols + nfp)
    ints, fp = ints.to(dev()), fp.to(dev())
    q_ref, meta_ref, fp_ref = ref.asym_quantize(x, ints, fp, bits)
    torch.cuda.synchronize()
    q, meta, fp_x = quik.asymmetric.quantize(x, ints, fp, bits)
    torch.cuda.synchronize()
    assert q.dtype == q_ref.dtype and q.shape == q_ref.shape
    assert torch.equal(meta, meta_ref)
    assert torch.equal(fp_x, fp_ref)
    assert torch.equal(q, q_ref)
    # the layer path's variant (16-bit ids, one code per byte) carries the same codes
    from quik_b200.qlinear import _to_u16
    qw, meta_w, _ = quik.asymmetric.quantize_u16(x, _to_u16(ints), _to_u16(fp), bits, True)
    assert torch.equal(meta_w, meta_ref)
    if bits == 8:
        assert torch.equal(qw, q_ref)
    else:
        lo = ((q_ref & 0xF).to(torch.int8) ^ 8) - 8
        hi = ((q_ref >> 4).to(torch.int8) ^ 8) - 8
        assert torch.equal(qw, torch.stack([lo, hi], dim=2).reshape(rows, -1))
    assert_device_clean()


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("rows,cols", [(37, 1024), (128, 4096), (2, 512)])
def test_find_meta_and_quantize_old_equal_reference_kernels(bits, rows, cols):
    import quik
    ref = ref_ops()
    x = _activations(rows, cols, torch.float16, rows * cols).to(dev())
    meta_ref = ref.asym_find_meta(x, bits)
    q_ref = ref.asym_quantize_old(x, meta_ref, bits)
    torch.cuda.synchronize()
    meta = quik.asymmetric.find_meta(x, bits)
    assert torch.equal(meta, meta_ref)
    assert torch.equal(quik.asymmetric.quantizeOld(x, meta_ref, bits), q_ref)
    assert_device_clean()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("rows,cols", [(37, 1000), (128, 4096), (2048, 264)])
def test_asym_dequantize_equals_reference_kernel(dtype, bits, rows, cols):
    """quik.asymmetric.dequantize (asymmetric.cu:119-233).  The reference source writes two roundings per product-sum
    (a * b, then + c); whether the compiler fuses them is its choice, so the fp32 intermediate may differ by a few of
    its last places relative to the largest term.  Identical bytes are demanded except for at most 1e-3 of the
    elements, which may differ by one unit in the last place of the output type plus that fp32 slack (it shows where
    the terms cancel)."""
    import quik
    ref = ref_ops()
    g = torch.Generator().manual_seed(rows * cols + bits)
    x = torch.randint(-200000, 200000, (rows, cols), generator=g, dtype=torch.int32).to(dev())
    meta = torch.stack([torch.rand(rows, generator=g) * 0.1 + 1e-3, torch.randn(rows, generator=g)], 1).reshape(-1).to(dtype).to(dev())
    sc = (torch.rand(cols, 1, generator=g) * 0.01 + 1e-4).to(dtype).to(dev())
    wr = torch.randn(1, cols, generator=g).to(dtype).to(dev())
    y = torch.randn(rows, cols, generator=g).to(dtype).to(dev())
    out_ref = ref.asym_dequantize(x, meta, sc, wr, y, bits)
    torch.cuda.synchronize()
    out = quik.asymmetric.dequantize(x, meta, sc, wr, y, bits)
    differ = out != out_ref
    frac = differ.float().mean().item()
    srow, zrow = meta[0::2].float().unsqueeze(1), meta[1::2].float().unsqueeze(1)
    shift = 8.0 if bits == 4 else 128.0
    terms = (x.float() * srow * sc.float().t()).abs() + ((zrow + shift * srow) * wr.float()).abs() + y.float().abs()
    slack = out_ref.float().abs() * (2.0 ** -10 if dtype == torch.float16 else 2.0 ** -7) + terms * 2.0 ** -21 + 1e-7
    worst = ((out.float() - out_ref.float()).abs() / slack).max().item()
    assert frac <= 1e-3 and worst <= 1.0, (frac, worst)
    assert_device_clean()


def test_symmetric_ops_equal_reference_kernels():
    import quik
    ref = ref_ops()
    torch.manual_seed(1)
    n, k, m = 512, 2048, 256
    src = torch.randn(n, k, dtype=torch.float16).to(dev())
    scale = (torch.rand(n, 1) * 0.05 + 0.01).half().to(dev())
    assert torch.equal(quik.symmetric.quantize(src, scale, 8), ref.sym_quantize_int8(src, scale))
    # The reference's 4-bit symmetric quantizer does not clamp: it hands round(x / scale) to CUTLASS's int4 type,
    # whose constructor (in the CUTLASS version of this image) asserts on the device that the value fits.  Only
    # values that round into [-8, 7] are fed to it.
    small = (torch.randn(n, k) * 2).clamp(-7.4, 7.4).half().to(dev())
    one = torch.ones(n, 1, dtype=torch.float16, device=dev())
    assert torch.equal(quik.symmetric.quantize(small, one, 4), ref.sym_quantize_int4(small, one))
    sr = torch.randn(m, 1, dtype=torch.float16).to(dev())
    sc = torch.randn(1, n, dtype=torch.float16).to(dev())
    y = torch.randn(m, n, dtype=torch.float16).to(dev())
    c = torch.randn(m, n, dtype=torch.float16).to(dev())
    assert torch.equal(quik.symmetric.dequantize(c, sr, sc, y, 16), ref.sym_dequantize_half(c, sr, sc, y))
    ci = torch.randint(-2000, 2000, (m, n), dtype=torch.int32, device=dev())
    assert torch.equal(quik.symmetric.dequantize(ci, sr, sc, y, 32), ref.sym_dequantize_int32(ci, sr, sc, y))
    c8 = torch.randint(-128, 128, (m, n), dtype=torch.int8, device=dev())
    assert torch.equal(quik.symmetric.dequantize(c8, sr, sc, y, 8), ref.sym_dequantize_int8(c8, sr, sc, y))
    assert_device_clean()


def _unpack_nibbles(p):
    """uint8 [R, C] of packed int4 (element 2j in the low nibble) -> int8 [R, 2C]."""
    lo = ((p & 0xF).to(torch.int8) ^ 8) - 8
    hi = ((p >> 4).to(torch.int8) ^ 8) - 8
    return torch.stack([lo, hi], dim=2).reshape(p.shape[0], -1)


@pytest.mark.parametrize("M,K,N,F,bits", [(16, 4352, 1024, 256, 4), (300, 4352, 1000, 256, 4), (2048, 4352, 2048, 256, 4),
                                          (64, 11264, 512, 256, 8), (2048, 11264, 1024, 256, 8)])
def test_layer_forward_vs_composition_of_reference_kernels(M, K, N, F, bits):
    """MixedQLinear.forward of the reference (experiments/qlinear.py:105-148) rebuilt from the reference's own
    kernels: its quantizer, an exact integer product in place of its CUTLASS GEMM (same integers by definition),
    torch's F.linear on the outlier columns as in the reference, its dequantize kernel.  The fused layer of this
    repository stays within the stated 1e-2 x RMS of it; the unfused operator sequence within a last place."""
    from quik_b200.workloads import make_layer
    ref = ref_ops()
    case = make_layer("t", M, K, N, bits, F=F, seed=M + N, device=dev(), clip=False)
    m, x = case.module, case.x
    q, meta, fp_x = ref.asym_quantize(x, m.int_indices, m.fp_indices, bits)
    qi = _unpack_nibbles(q) if bits == 4 else q
    wi = _unpack_nibbles(m.int_weight) if bits == 4 else m.int_weight
    acc = (qi.double() @ wi.double().t()).to(torch.int32)            # exact: |sum| < 2^53
    fp_result = torch.nn.functional.linear(fp_x, m.fp_weight, m.bias)
    out_ref = ref.asym_dequantize(acc, meta, m.weights_scales, m.reduced_w, fp_result, bits)
    torch.cuda.synchronize()
    fused = m(x.unsqueeze(0))[0]
    assert rel_rms_err(fused, out_ref) < 1e-2
    m.fused = False
    unfused = m(x.unsqueeze(0))[0]
    m.fused = True
    assert rel_rms_err(unfused, out_ref) < 2e-3
    assert_device_clean()


def _pack_i4(v):
    """int8 [R, C] of codes in [-8, 7] -> uint8 [R, C/2], element 2j in the low nibble."""
    u = (v.to(torch.int16) & 0xF).to(torch.uint8)
    return (u[:, 0::2] | (u[:, 1::2] << 4)).contiguous()


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("M,N,K", [(128, 256, 1024), (300, 520, 2048), (2048, 4096, 4096), (1, 128, 11008), (2048, 1024, 11008)])
def test_int_matmul_equals_reference_cutlass_gemm(bits, M, N, K):
    """quik.matmul.int4Matmul / int8Matmul against the reference's CUTLASS GEMMs (matmul.cu:17-55,98-136): the same
    int32 values, bit for bit."""
    import quik
    ref = ref_ops()
    g = torch.Generator().manual_seed(M + N + K + bits)
    lo, hi = (-8, 8) if bits == 4 else (-128, 128)
    a = torch.randint(lo, hi, (M, K), generator=g, dtype=torch.int8).to(dev())
    b = torch.randint(lo, hi, (N, K), generator=g, dtype=torch.int8).to(dev())
    if bits == 4:
        a, b = _pack_i4(a), _pack_i4(b)
        c_ref = ref.int4_matmul(a, b)
        torch.cuda.synchronize()
        c = quik.matmul.int4Matmul(a, b)
    else:
        c_ref = ref.int8_matmul(a, b)
        torch.cuda.synchronize()
        c = quik.matmul.int8Matmul(a, b)
    assert c.dtype == c_ref.dtype and torch.equal(c, c_ref)
    assert_device_clean()


@pytest.mark.parametrize("bits", [4, 8])
def test_fused_dequantize_ops_vs_reference_fused_kernels(bits):
    """The reference's fused GEMM + dequantize ops (asymmetric and symmetric fused_dequantize.cu) on the data of its
    own test (test/python/test_fused.py:40-67).  The reference evaluates the epilogue in fp16, this repository in
    fp32 with one rounding: agreement within three fp16 units of the largest term."""
    import quik
    ref = ref_ops()
    M, N, K = 1024, 5120, 2048
    g = torch.Generator().manual_seed(2)
    a_i = torch.randint(-3, 3, (M, K), generator=g, dtype=torch.int8).to(dev())
    b_i = torch.randint(-3, 3, (N, K), generator=g, dtype=torch.int8).to(dev())
    a, b = (_pack_i4(a_i), _pack_i4(b_i)) if bits == 4 else (a_i, b_i)
    sr = torch.rand(M, 1, generator=g).half().to(dev())
    sc = torch.rand(1, N, generator=g).half().to(dev())
    zr = torch.rand(M, 1, generator=g).half().to(dev())
    wr = torch.rand(1, N, generator=g).half().to(dev())
    y = torch.rand(M, N, generator=g).half().to(dev())
    sv = 0.4376
    if bits == 4:
        out_ref = ref.asym_int4_fused_dequantize(a, b, sr, sc, sv, zr, wr, y)
        outs_ref = ref.sym_int4_fused_dequantize(a, b, sr, sc, y)
        torch.cuda.synchronize()
        out = quik.asymmetric.int4FusedDequantize(a, b, sr, sc, sv, zr, wr, y)
        outs = quik.symmetric.int4FusedDequantize(a, b, sr, sc, y)
    else:
        out_ref = ref.asym_int8_fused_dequantize(a, b, sr, sc, sv, zr, wr, y)
        outs_ref = ref.sym_int8_fused_dequantize(a, b, sr, sc, y)
        torch.cuda.synchronize()
        out = quik.asymmetric.int8FusedDequantize(a, b, sr, sc, sv, zr, wr, y)
        outs = quik.symmetric.int8FusedDequantize(a, b, sr, sc, y)
    acc = (a_i.double() @ b_i.double().t()).float()
    t1 = (acc * sr.float() * sc.float()).abs()
    t2 = ((zr.float() + sv * sr.float()) * wr.float()).abs()
    ulp = torch.maximum(torch.maximum(t1, t2), torch.maximum(y.float().abs(), out_ref.float().abs())) * 2 ** -10
    assert ((out.float() - out_ref.float()).abs() <= 3 * ulp).all()
    ulp_s = torch.maximum(torch.maximum(t1, y.float().abs()), outs_ref.float().abs()) * 2 ** -10
    assert ((outs.float() - outs_ref.float()).abs() <= 3 * ulp_s).all()
    assert_device_clean()


def _reference_forward(ref, m, x, bits):
    """MixedQLinear.forward of the reference (experiments/qlinear.py:105-148), op for op, on the reference's kernels."""
    q, meta, fp_x = ref.asym_quantize(x, m.int_indices, m.fp_indices, bits)
    fp_result = torch.nn.functional.linear(fp_x, m.fp_weight, m.bias)
    acc = ref.int4_matmul(q, m.int_weight) if bits == 4 else ref.int8_matmul(q, m.int_weight)
    return ref.asym_dequantize(acc, meta, m.weights_scales, m.reduced_w, fp_result, bits)


@pytest.mark.parametrize("M,K,N,F,bits", [(16, 4352, 1024, 256, 4), (128, 4352, 4096, 256, 4), (2048, 4352, 4096, 256, 4),
                                          (64, 11264, 512, 256, 8), (2048, 11264, 4096, 256, 8)])
def test_layer_forward_vs_reference_forward(M, K, N, F, bits):
    """The whole reference layer on the reference's own kernels (quantize, CUTLASS GEMM, F.linear, dequantize)
    against this repository's fused layer: max-abs difference below 1e-2 of the output RMS."""
    from quik_b200.workloads import make_layer
    ref = ref_ops()
    case = make_layer("t", M, K, N, bits, F=F, seed=M + N, device=dev(), clip=False)
    out_ref = _reference_forward(ref, case.module, case.x, bits)
    torch.cuda.synchronize()
    out = case.module(case.x.unsqueeze(0))[0]
    assert rel_rms_err(out, out_ref) < 1e-2
    assert_device_clean()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bits", [4, 8])
def test_cpu_oracle_matches_reference_kernels(dtype, bits):
    """The CPU oracle itself (oracle/kernel_path.py) against the reference's kernels: quantizer codes exact except at
    most 1e-5 of the codes off by one (the device's reciprocal-based half division against an IEEE division), meta and
    outlier columns exact, dequantize exact up to the same fused-multiply-add freedom as the kernels, layer forward
    within 1e-2 x RMS."""
    from oracle import kernel_path as kp
    from quik_b200.workloads import make_layer
    ref = ref_ops()
    rows, cols, nfp = 64, 4352, 256
    x = _activations(rows, cols, dtype, 11 + bits)
    ints, fp = _indices(cols, nfp, "ascending", 3)
    q_ref, meta_ref, fp_ref = ref.asym_quantize(x.to(dev()), ints.to(dev()), fp.to(dev()), bits)
    q, meta, fp_x = kp.asym_quantize(x, ints, fp, bits)
    assert torch.equal(meta, meta_ref.cpu()) and torch.equal(fp_x, fp_ref.cpu())
    codes = _unpack_nibbles(q) if bits == 4 else q
    codes_ref = _unpack_nibbles(q_ref.cpu()) if bits == 4 else q_ref.cpu()
    diff = (codes.to(torch.int16) - codes_ref.to(torch.int16)).abs()
    assert diff.max() <= 1 and (diff != 0).float().mean() <= 1e-5
    if dtype == torch.float16:
        case = make_layer("t", 64, 4352, 512, bits, F=256, seed=5, device=dev(), clip=False)
        m = case.module
        buf = {"int_weight": m.int_weight.cpu(), "weights_scales": m.weights_scales.cpu(), "reduced_w": m.reduced_w.cpu(),
               "int_indices": m.int_indices.cpu(), "fp_indices": m.fp_indices.cpu(), "fp_weight": m.fp_weight.cpu(), "bias": None}
        out_oracle = kp.mixed_linear_forward(case.x.cpu(), buf, bits, round_y=True)
        out_ref = _reference_forward(ref, m, case.x, bits)
        assert rel_rms_err(out_oracle, out_ref.cpu()) < 1e-2
    assert_device_clean()


def test_timing_against_reference_kernels(capsys):
    """Not a parity check: times the reference's quantize and dequantize kernels next to this repository's on the
    7B layer inputs (2048 tokens) and prints the figures (run with -s).  CUDA events around 20 replays of a graph of 8
    launches over rotating inputs larger than L2."""
    import quik
    from quik_b200.qlinear import _to_u16
    ref = ref_ops()
    lines = []
    for cols, nfp, bits in ((4352, 256, 4), (11264, 256, 8)):
        xs = [_activations(2048, cols, torch.float16, i).to(dev()) for i in range(8)]
        ints, fp = _indices(cols, nfp, "ascending", 1)
        ints, fp = ints.to(dev()), fp.to(dev())
        i16, f16 = _to_u16(ints), _to_u16(fp)

        def timed(fn, graph):
            # The reference's kernels launch on the legacy default stream whatever the current stream is, so they
            # cannot be captured: they are timed eagerly (their kernels are much longer than a launch).  This
            # repository's are also replayed from a CUDA graph, which takes the host's launch cost out.
            for x in xs:
                fn(x)
            torch.cuda.synchronize()
            if not graph:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(20):
                    for x in xs:
                        fn(x)
                b.record()
                torch.cuda.synchronize()
                return a.elapsed_time(b) * 1e3 / 160
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                for x in xs:
                    fn(x)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    for x in xs:
                        fn(x)
                g.replay()
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(20):
                    g.replay()
                b.record()
                torch.cuda.synchronize()
            return a.elapsed_time(b) * 1e3 / 160

        t_ref = timed(lambda x: ref.asym_quantize(x, ints, fp, bits), False)
        t_eager = timed(lambda x: quik.asymmetric.quantize_u16(x, i16, f16, bits, True), False)
        t_graph = timed(lambda x: quik.asymmetric.quantize_u16(x, i16, f16, bits, True), True)
        lines.append(f"quantize [2048, {cols}] {bits}-bit: reference kernel {t_ref:.1f} us (eager), this repository "
                     f"{t_eager:.1f} us (eager, host bound) / {t_graph:.1f} us (graph replay)")
    n = 4096
    acc = torch.randint(-200000, 200000, (2048, n), dtype=torch.int32, device=dev())
    meta = (torch.rand(4096, device=dev()) * 0.1 + 1e-3).half()
    sc = (torch.rand(n, 1, device=dev()) * 0.01 + 1e-4).half()
    wr = torch.randn(1, n, device=dev()).half()
    y = torch.randn(2048, n, device=dev()).half()
    for name, fn in (("reference kernel", lambda: ref.asym_dequantize(acc, meta, sc, wr, y, 4)),
                     ("this repository (discrete op; the layer fuses it into the GEMM)", lambda: quik.asymmetric.dequantize(acc, meta, sc, wr, y, 4))):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(50):
            fn()
        b.record()
        torch.cuda.synchronize()
        lines.append(f"dequantize [2048, {n}]: {name} {a.elapsed_time(b) * 1e3 / 50:.1f} us")
    # whole layers: the reference's operator sequence on its own kernels (eager; they cannot be captured) against this
    # repository's fused layer (eager and replayed from a graph)
    from quik_b200.workloads import make_layer
    for name, K, N, bits in (("qkv", 4352, 12288, 4), ("o", 4352, 4096, 4), ("gate+up", 4352, 22016, 4), ("down", 11264, 4096, 8)):
        case = make_layer(name, 2048, K, N, bits, F=256, seed=0, device=dev(), clip=False)
        m, x = case.module, case.x

        def run_ref():
            return _reference_forward(ref, m, x, bits)

        def run_ours():
            return m(x.unsqueeze(0))

        times = []
        for fn in (run_ref, run_ours):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(10):
                fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3 / 10)
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            run_ours()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                run_ours()
            g.replay()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(10):
                g.replay()
            b.record()
            torch.cuda.synchronize()
        ops = 2.0 * 2048 * N * K
        lines.append(f"layer {name} [2048 x {K}] -> {N}, {bits}-bit: reference kernels {times[0]:.0f} us ({ops / times[0] / 1e6:.0f} TOPS), "
                     f"this repository {times[1]:.0f} us eager / {a.elapsed_time(b) * 100:.0f} us graph "
                     f"({ops / (a.elapsed_time(b) * 100) / 1e6:.0f} TOPS)")
        del case, m, x
        torch.cuda.empty_cache()
    with capsys.disabled():
        print()
        for line in lines:
            print("  " + line)
    assert_device_clean()
