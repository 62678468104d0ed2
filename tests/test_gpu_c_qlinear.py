"""GPU parity: MixedQLinear.forward (fused, unfused, shared input, small-M, bf16) vs the CPU oracle."""
import pytest
import torch

from oracle import kernel_path as kp
from quik_b200 import _lib
from quik_b200.qlinear import MixedQLinear, SharedQuantizedInput
from quik_b200.workloads import make_layer
from tests.gpu_util import assert_device_clean, dev, rel_rms_err

pytestmark = pytest.mark.gpu

# BASELINE tolerance: max-abs error of the fp16 output relative to the output RMS
TOL_RMS = 1e-2


def _oracle_out(case, round_y):
    m = case.module
    buf = {"int_weight": m.int_weight.cpu(), "weights_scales": m.weights_scales.cpu(), "reduced_w": m.reduced_w.cpu(),
           "int_indices": m.int_indices.cpu(), "fp_indices": m.fp_indices.cpu(),
           "bias": None if m.bias is None else m.bias.cpu()}
    if m.fp_features_num > 0:
        buf["fp_weight"] = m.fp_weight.cpu()
    return kp.mixed_linear_forward(case.x.cpu(), buf, m.bits, round_y=round_y)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,K,N,F,bits", [
    (1, 4096, 512, 256, 4), (16, 4096, 264, 256, 4), (16, 1024, 128, 0, 8), (7, 11008, 256, 256, 8),
    (17, 4096, 512, 256, 4), (129, 4096, 520, 256, 4), (256, 1024, 384, 0, 4), (128, 11008, 256, 256, 8),
    (2048, 4096, 1024, 256, 4), (300, 8192, 1024, 1024, 4), (64, 96, 40, 32, 4),
    (40, 112, 24, 32, 4), (9, 112, 24, 32, 4),      # 80 integer columns: packed rows of 40 bytes, tiled GEMM at any M
])
def test_fused_forward_matches_oracle(dtype, M, K, N, F, bits):
    case = make_layer("t", M, K, N, bits, F=F, seed=M + N, device=dev(), dtype=dtype, clip=False)
    out = case.module(case.x.unsqueeze(0))
    assert out.shape == (1, M, N) and out.dtype == dtype
    ref = _oracle_out(case, round_y=False)
    err = rel_rms_err(out[0].cpu(), ref)
    # bf16 has 3 fewer mantissa bits: the final rounding and the storage-type rounding of the outlier
    # product are each worth up to 2^-8 of the value
    tol = TOL_RMS if dtype == torch.float16 else 4e-2
    assert err < tol, err
    # the reference's own unfused sequence rounds the outlier product to the storage type before the
    # dequantize step; in bf16 that extra rounding alone is worth up to 2^-8 of |y|
    ref_rounded = _oracle_out(case, round_y=True)
    assert rel_rms_err(out[0].cpu(), ref_rounded) < tol
    out2 = case.module(case.x.unsqueeze(0))
    assert torch.equal(out, out2)                            # deterministic
    assert_device_clean()


@pytest.mark.parametrize("col_pad", [8, 3])
@pytest.mark.parametrize("engine", [_lib.ENGINE_TCGEN05, _lib.ENGINE_TCGEN05_TS], ids=["smem_operands", "tmem_operand"])
@pytest.mark.parametrize("tile,pair", [(0, 0), (240, 2), (144, 2), (176, 1)])
@pytest.mark.parametrize("M,K,N,F,bits", [(300, 1088, 520, 64, 4), (129, 1088, 264, 64, 8), (257, 608, 1000, 32, 4),
                                          (16, 1088, 520, 64, 4), (100, 1088, 520, 64, 8)])
def test_fused_layer_writes_only_its_columns(M, K, N, F, bits, tile, pair, engine, col_pad):
    """The layer's output is a window of a poisoned slab (rows and columns of padding on every side, handed over as
    `out_buffer` with a row pitch wider than N): the window equals the plain forward bit for bit and the padding is
    untouched.  col_pad = 8 keeps the window 16-byte aligned (vector stores, parked outlier products in the
    permuted layout), col_pad = 3 does not (scalar stores); the tile widths end a warp's column range with a
    16-column step.  Covers the ragged-edge stores and the parked-tile writes of the tiled kernel and the stores of
    the weight-streaming engines (16 and 100 tokens)."""
    case = make_layer("t", M, K, N, bits, F=F, seed=M + N, device=dev(), clip=False)
    row_pad = 5
    poison = -1234.0
    try:
        _lib.set_engine(engine)
        _lib.set_tile_n(tile)
        _lib.set_cta_pair(pair)
        want = case.module(case.x.unsqueeze(0))[0].clone()
        slab = torch.full((M + 2 * row_pad, N + 2 * col_pad), poison, dtype=torch.float16, device=dev())
        window = slab[row_pad:row_pad + M, col_pad:col_pad + N]
        case.module.out_buffer = window
        got = case.module(case.x.unsqueeze(0))[0]
        assert got.data_ptr() == window.data_ptr()
        torch.cuda.synchronize()
    finally:
        case.module.out_buffer = None
        _lib.set_engine(_lib.ENGINE_AUTO)
        _lib.set_tile_n(0)
        _lib.set_cta_pair(0)
    assert_device_clean()
    assert torch.equal(window, want)
    border = slab.clone()
    border[row_pad:row_pad + M, col_pad:col_pad + N] = poison
    assert bool((border == poison).all()), "the layer wrote outside its [M, N] window"
    assert rel_rms_err(want.cpu(), _oracle_out(case, round_y=False)) < TOL_RMS


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,K,N,F,bits", [
    (16, 256, 128, 0, 4), (16, 1280, 128, 256, 8), (1, 4352, 512, 256, 4), (16, 4352, 264, 256, 4), (7, 11264, 256, 256, 8),
    (16, 4352, 4096, 256, 4),      # K split over a cluster of 4 CTAs
    (13, 11264, 4096, 256, 8),     # ... of 8
    (16, 4352, 22016, 256, 4),     # one CTA per slab, more slabs than fit at once
    (5, 4232, 300, 72, 4),         # ragged N, K and F
])
def test_small_m_engines_agree(dtype, M, K, N, F, bits):
    """Few tokens: the three weight-streaming engines (tcgen05 with on-chip widening; mma.sync fed by direct loads or
    by a TMA ring) and the tensor-core GEMM on widened weights give the oracle's result; the integer part is exact
    in all of them."""
    case = make_layer("t", M, K, N, bits, F=F, seed=M + N, device=dev(), dtype=dtype, clip=False)
    outs = {}
    try:
        for mode in (_lib.SMALL_M_TCGEN05, _lib.SMALL_M_MMA_SYNC, _lib.SMALL_M_TMA_MMA, _lib.SMALL_M_OFF, _lib.SMALL_M_AUTO):
            _lib.set_small_m(mode)
            outs[mode] = case.module(case.x.unsqueeze(0))[0].clone()
            again = case.module(case.x.unsqueeze(0))[0]
            assert torch.equal(outs[mode], again)                # deterministic (split-K included)
    finally:
        _lib.set_small_m(_lib.SMALL_M_AUTO)
    assert_device_clean()
    ref = _oracle_out(case, round_y=False)
    tol = TOL_RMS if dtype == torch.float16 else 4e-2
    for mode, out in outs.items():
        assert rel_rms_err(out.cpu(), ref) < tol, mode
    # the engines differ only in the summation order of the outlier product: at most one unit in the last place of
    # the largest outputs (2^-10 of 4 x RMS in fp16)
    agree = 5e-3 if dtype == torch.float16 else 4e-2
    assert rel_rms_err(outs[_lib.SMALL_M_TCGEN05], outs[_lib.SMALL_M_MMA_SYNC]) < agree
    assert rel_rms_err(outs[_lib.SMALL_M_TCGEN05], outs[_lib.SMALL_M_OFF]) < agree
    assert rel_rms_err(outs[_lib.SMALL_M_TMA_MMA], outs[_lib.SMALL_M_MMA_SYNC]) < agree
    if F == 0:
        assert torch.equal(outs[_lib.SMALL_M_TCGEN05], outs[_lib.SMALL_M_MMA_SYNC])
        assert torch.equal(outs[_lib.SMALL_M_TMA_MMA], outs[_lib.SMALL_M_MMA_SYNC])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M", [17, 33, 64, 65, 100, 128])
@pytest.mark.parametrize("K,N,F,bits", [(4352, 4096, 256, 4), (11264, 520, 256, 8), (1056, 300, 32, 4)])
def test_streaming_engine_up_to_128_tokens(dtype, M, K, N, F, bits):
    """17 to 128 tokens run on the tcgen05 weight-streaming engine (token operand of 64 or 128 rows, weights in
    storage format); same result as the tiled tensor-core GEMM on widened weights, and the oracle's."""
    case = make_layer("t", M, K, N, bits, F=F, seed=M + N, device=dev(), dtype=dtype, clip=False)
    try:
        out = case.module(case.x.unsqueeze(0))[0].clone()
        again = case.module(case.x.unsqueeze(0))[0]
        _lib.set_small_m(_lib.SMALL_M_OFF)
        tiled = case.module(case.x.unsqueeze(0))[0].clone()
    finally:
        _lib.set_small_m(_lib.SMALL_M_AUTO)
    assert_device_clean()
    assert torch.equal(out, again)
    tol = TOL_RMS if dtype == torch.float16 else 4e-2
    assert rel_rms_err(out.cpu(), _oracle_out(case, round_y=False)) < tol
    assert rel_rms_err(out, tiled) < (5e-3 if dtype == torch.float16 else 4e-2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,K,N,F,bits", [(129, 1088, 520, 64, 4), (300, 4352, 1024, 256, 4), (2048, 4096, 1280, 256, 4),
                                          (257, 11264, 520, 256, 8), (513, 1024, 264, 0, 4), (400, 2080, 96, 32, 8),
                                          (1000, 4128, 4096, 32, 4)])
def test_tensor_memory_operand_engine_matches_shared_memory_engine(dtype, M, K, N, F, bits):
    """The two tcgen05 engines (token codes one per byte from shared memory; packed 4-bit codes widened on chip into
    tensor memory) compute every output element from the same exact integer sum and the same order of outlier
    products, so their results are identical bit for bit whatever tiles they pick; both match the oracle."""
    case = make_layer("t", M, K, N, bits, F=F, seed=M + N, device=dev(), dtype=dtype, clip=False)
    outs = {}
    try:
        for eng in (_lib.ENGINE_TCGEN05, _lib.ENGINE_TCGEN05_TS):
            _lib.set_engine(eng)
            outs[eng] = case.module(case.x.unsqueeze(0))[0].clone()
            assert torch.equal(outs[eng], case.module(case.x.unsqueeze(0))[0])
    finally:
        _lib.set_engine(_lib.ENGINE_AUTO)
    assert_device_clean()
    assert torch.equal(outs[_lib.ENGINE_TCGEN05], outs[_lib.ENGINE_TCGEN05_TS])
    tol = TOL_RMS if dtype == torch.float16 else 4e-2
    assert rel_rms_err(outs[_lib.ENGINE_TCGEN05_TS].cpu(), _oracle_out(case, round_y=False)) < tol


@pytest.mark.parametrize("M", [16, 300])
def test_dependent_launch_matches_stream_order(M):
    """A chain of layers (each output feeds the next quantizer) with kernels launched as programmatic dependents
    gives bit-identical results to plain stream order, eagerly and replayed from a CUDA graph."""
    cases = [make_layer(f"l{i}", M, 1024 + 64, 1024 + 64, 4 if i % 2 == 0 else 8, F=64, seed=i, device=dev(), clip=False)
             for i in range(4)]
    x0 = cases[0].x

    def chain():
        h = x0
        for c in cases:
            h = c.module(h.unsqueeze(0))[0]
            h = (h / h.float().abs().max().clamp_min(1e-3)).to(x0.dtype)     # keep magnitudes stable (a torch kernel in between)
        return h

    try:
        _lib.set_pdl(False)
        ref = chain().clone()
        _lib.set_pdl(True)
        eager = chain().clone()
        torch.cuda.synchronize()
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                out = chain()
            for _ in range(3):
                g.replay()
        torch.cuda.synchronize()
    finally:
        _lib.set_pdl(True)
    assert torch.equal(eager, ref)
    assert torch.equal(out, ref)
    assert_device_clean()


def test_dependent_launch_back_to_back_layers():
    """Layers launched back to back with no other kernel in between (shared quantized input: quantizer, then three
    fused launches), where a launch can overtake its predecessor's tail; outputs equal plain stream order."""
    shared = SharedQuantizedInput(3)
    cases = [make_layer(f"m{i}", 16, 4096 + 256, 1024, 4, F=256, seed=0, device=dev(), shared_input=shared, clip=False)
             for i in range(3)]
    x = cases[0].x
    res = {}
    try:
        for on in (False, True):
            _lib.set_pdl(on)
            for rep in range(3):
                res[on] = [c.module(x.unsqueeze(0)).clone() for c in cases]
        torch.cuda.synchronize()
    finally:
        _lib.set_pdl(True)
    for a, b in zip(res[False], res[True]):
        assert torch.equal(a, b)
    assert_device_clean()


@pytest.mark.parametrize("pair", [1, 2])
@pytest.mark.parametrize("M,K,N,F,bits", [(300, 4096, 520, 256, 4), (2048, 4096, 2048, 256, 4), (640, 11008, 512, 256, 8),
                                          (128, 1024, 256, 64, 4), (513, 2048, 1000, 0, 4)])
def test_fused_forward_single_cta_and_pair_agree(pair, M, K, N, F, bits):
    """Both tile schedules (one CTA per tile, CTA pair per 256-row tile) against the oracle and each other."""
    case = make_layer("t", M, K, N, bits, F=F, seed=7, device=dev(), clip=False)
    _lib.set_cta_pair(pair)
    try:
        out = case.module(case.x.unsqueeze(0))[0]
        torch.cuda.synchronize()
    finally:
        _lib.set_cta_pair(0)
    assert_device_clean()
    ref = _oracle_out(case, round_y=True)
    assert rel_rms_err(out.cpu(), ref) < TOL_RMS
    _lib.set_cta_pair(1)
    try:
        single = case.module(case.x.unsqueeze(0))[0]
    finally:
        _lib.set_cta_pair(0)
    assert rel_rms_err(out.cpu(), single.cpu()) < 2e-3      # only the outlier product's summation order differs


@pytest.mark.parametrize("M,bits,F", [(64, 4, 256), (5, 8, 0), (200, 8, 256)])
def test_unfused_forward_matches_oracle(M, bits, F):
    case = make_layer("t", M, 4096, 256, bits, F=F, seed=3, device=dev(), clip=False)
    case.module.fused = False
    out = case.module(case.x.unsqueeze(0))[0].cpu()
    ref = _oracle_out(case, round_y=True)
    # same int32 accumulators and same fp32 epilogue; only the cuBLAS outlier GEMM may round differently
    assert rel_rms_err(out, ref) < 2e-3
    case.module.fused = True
    fused = case.module(case.x.unsqueeze(0))[0].cpu()
    assert rel_rms_err(fused, out) < TOL_RMS


def test_bias_and_no_outliers():
    torch.manual_seed(0)
    K, N, M = 512, 128, 40
    lin = torch.nn.Linear(K, N, bias=True)
    w = (0.02 * torch.randn(N, K)).half()
    scales = w.float().abs().max(1, keepdim=True)[0] / 7
    mod = MixedQLinear.from_float(lin, w, scales, fp_indices=None, bits=4).to(dev())
    x = torch.randn(M, K).half().to(dev())
    out = mod(x.unsqueeze(0))[0].cpu()
    buf = kp.from_float_buffers(w, scales, None, 4, bias=lin.bias.data.half())
    ref = kp.mixed_linear_forward(x.cpu(), buf, 4, round_y=True, contract=True)
    # no outlier GEMM: exact integer GEMM + the fp32 multiply-add epilogue -> same fp16 values
    diff = (out.float() - ref.float()).abs()
    assert (diff <= ref.float().abs() * 2 ** -10 + 2.0 ** -24).all() and (diff != 0).float().mean() < 1e-4
    for name in ("int_weight", "weights_scales", "reduced_w", "int_indices", "bias"):
        assert torch.equal(getattr(mod, name).cpu(), buf[name]), name


def test_shared_quantized_input_groups():
    """q/k/v style group of three layers shares one quantizer call (experiments/llama.py:402-411)."""
    shared = SharedQuantizedInput(3)
    cases = [make_layer(f"m{i}", 48, 1024, 128, 4, F=64, seed=0, device=dev(), shared_input=shared, clip=False)
             for i in range(3)]
    x = cases[0].x
    outs = []
    for i, c in enumerate(cases):
        outs.append(c.module(x.unsqueeze(0)))
        if i < 2:
            assert shared.qint_x is not None and shared.cur_group_elem == i + 1
    assert shared.qint_x is None and shared.cur_group_elem == 0
    for c, o in zip(cases, outs):
        solo = make_layer("s", 48, 1024, 128, 4, F=64, seed=0, device=dev(), clip=False)
        assert torch.equal(o, solo.module(x.unsqueeze(0)))


def test_state_dict_round_trip():
    case = make_layer("t", 32, 1024, 128, 4, F=64, seed=1, device=dev(), clip=False)
    sd = case.module.state_dict()
    fresh = MixedQLinear(1024, 128, fp_features_num=64, bits=4)
    fresh.bias = None
    fresh.load_state_dict(sd)
    fresh = fresh.to(dev())
    assert torch.equal(fresh(case.x.unsqueeze(0)), case.module(case.x.unsqueeze(0)))


def test_symmetric_branch_runs():
    torch.manual_seed(0)
    K, N, M = 256, 64, 16
    lin = torch.nn.Linear(K, N, bias=False)
    w = torch.randint(-7, 8, (N, K)).half()
    mod = MixedQLinear.from_float(lin, w, torch.ones(N, 1), fp_indices=None, symm=True, bits=4).to(dev())
    x = torch.randn(M, K).half().to(dev())
    out = mod(x.unsqueeze(0))[0].cpu()
    qs = (x.abs().max(1)[0].unsqueeze(1) / (1 << (4 - 1) - 1)).half().cpu()
    q = kp.sym_quantize(x.cpu(), qs, 4)
    acc = kp.int4_matmul(q, kp.pack_to_i4(w.to(torch.int8)))
    ref = kp.sym_dequantize(acc, qs, torch.ones(1, N).half(), torch.zeros(M, N).half(), 32)
    assert torch.equal(out, ref)


@pytest.mark.parametrize("bits,K,F", [(4, 4352, 256), (8, 2304, 256)])
def test_engines_agree_on_the_same_rows_across_token_counts(bits, K, F):
    """16, 128 and 129 tokens take three different engines (mma.sync streaming, tcgen05 streaming, tiled tcgen05
    GEMM).  The integer part is exact in all of them; the tiled engine rounds (outlier product + bias) to the storage
    type before the dequantize step (as the reference's F.linear output is rounded, experiments/qlinear.py:124) while
    the streaming engines keep it in fp32, so the same token differs by at most a couple of units in the last place of
    the largest outputs: 5e-3 of the output RMS in fp16."""
    N = 520
    case = make_layer("t", 129, K, N, bits, F=F, seed=11, device=dev(), clip=False)
    outs = {}
    for M in (16, 128, 129):
        outs[M] = case.module(case.x[:M].contiguous().unsqueeze(0))[0]
    assert_device_clean()
    ref = _oracle_out(case, round_y=False)
    for M, out in outs.items():
        assert rel_rms_err(out.cpu(), ref[:M]) < TOL_RMS, M
    assert rel_rms_err(outs[128][:16], outs[16]) < 5e-3
    assert rel_rms_err(outs[129][:128], outs[128]) < 5e-3


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_layers_on_two_devices_of_one_process():
    """One process driving layers on cuda:0 and cuda:1 in turn (the reference's llama_multigpu places layers this way,
    experiments/llama.py:295-326): shared-memory opt-ins and occupancy answers are kept per device.  Plain launches,
    no peer memory."""
    outs = []
    for d in (0, 1, 0, 1):
        device = torch.device("cuda", d)
        for M in (16, 300):
            case = make_layer("t", M, 1088, 520, 4, F=64, seed=5, device=device, clip=False)
            out = case.module(case.x.unsqueeze(0))
            torch.cuda.synchronize(device)
            assert out.device == device
            assert rel_rms_err(out[0].cpu(), _oracle_out(case, round_y=False)) < TOL_RMS
            with torch.cuda.device(device):
                assert _lib.device_status() == 0
            outs.append((M, out[0].cpu()))
    assert torch.equal(outs[0][1], outs[2][1]) and torch.equal(outs[1][1], outs[3][1])      # cuda:0 == cuda:1
