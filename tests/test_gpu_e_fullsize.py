"""GPU parity at the full BASELINE sizes.  The layer is row-separable (every output row depends only on
its own activation row), so the GPU runs the whole [M, K] problem and the CPU oracle re-computes a random
sample of rows end to end (quantizer, exact integer GEMM, dequantize); the sampled rows must agree within
the stated tolerance and the sampled quantizer bytes exactly."""
import pytest
import torch

from oracle import kernel_path as kp
from quik_b200 import asymmetric
from quik_b200.qlinear import _to_u16
from quik_b200.workloads import LLAMA2_70B, LLAMA2_7B, make_layer
from tests.gpu_util import assert_device_clean, dev, rel_rms_err

pytestmark = pytest.mark.gpu
TOL_RMS = 1e-2


def _buffers(m):
    buf = {"int_weight": m.int_weight.cpu(), "weights_scales": m.weights_scales.cpu(), "reduced_w": m.reduced_w.cpu(),
           "int_indices": m.int_indices.cpu(), "fp_indices": m.fp_indices.cpu(),
           "bias": None if m.bias is None else m.bias.cpu()}
    if m.fp_features_num > 0:
        buf["fp_weight"] = m.fp_weight.cpu()
    return buf


def _check_sampled_rows(case, n_rows=48, seed=0):
    out = case.module(case.x.unsqueeze(0))[0]
    torch.cuda.synchronize()
    assert_device_clean()
    g = torch.Generator().manual_seed(seed)
    rows = torch.randperm(case.M, generator=g)[:min(n_rows, case.M)].sort()[0]
    x_rows = case.x[rows.to(case.x.device)].cpu()
    ref = kp.mixed_linear_forward(x_rows, _buffers(case.module), case.bits, round_y=True, contract=True)
    got = out[rows.to(out.device)].cpu()
    assert rel_rms_err(got, ref) < TOL_RMS
    # quantizer bytes of the sampled rows: exact meta / outliers, codes equal up to the documented rare off-by-one
    m = case.module
    q, meta, fp_x = asymmetric.quantize(case.x, m.int_indices, m.fp_indices, case.bits)
    q_ref, meta_ref, fp_ref = kp.asym_quantize(x_rows, m.int_indices.cpu(), m.fp_indices.cpu(), case.bits)
    r = rows.to(q.device)
    assert torch.equal(meta.view(-1, 2)[r].cpu().reshape(-1), meta_ref)
    assert torch.equal(fp_x[r].cpu(), fp_ref)
    a = kp.unpack_i4(q[r].cpu()) if case.bits == 4 else q[r].cpu()
    b = kp.unpack_i4(q_ref) if case.bits == 4 else q_ref
    diff = (a.to(torch.int16) - b.to(torch.int16)).abs()
    assert diff.max() <= 1 and (diff != 0).float().mean() <= 1e-5


def test_config0_full_compare():
    """BASELINE config 0: M=2048, K=N=4096, F=256, 4-bit -- every output element against the oracle."""
    case = make_layer("cfg0", 2048, 4096, 4096, 4, F=256, seed=0, device=dev())
    out = case.module(case.x.unsqueeze(0))[0].cpu()
    ref = kp.mixed_linear_forward(case.x.cpu(), _buffers(case.module), 4, round_y=True, contract=True)
    assert rel_rms_err(out, ref) < TOL_RMS
    assert_device_clean()


@pytest.mark.parametrize("name,K,N,bits", LLAMA2_7B)
@pytest.mark.parametrize("M", [1, 16, 128, 2048])
def test_llama7b_shapes(name, K, N, bits, M):
    """BASELINE config 1: the 7B sweep, all four layer shapes x M in {1, 16, 128, 2048}."""
    _check_sampled_rows(make_layer(name, M, K, N, bits, F=256, seed=1, device=dev(), clip=False))


@pytest.mark.parametrize("name,K,N,bits", LLAMA2_70B)
def test_llama70b_shapes(name, K, N, bits):
    """BASELINE config 3 on one GPU: 70B shapes at M=4096."""
    _check_sampled_rows(make_layer(name, 4096, K, N, bits, F=256, seed=2, device=dev(), clip=False), n_rows=24)
    torch.cuda.empty_cache()


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("F", [0, 128, 256, 512, 1024])
@pytest.mark.parametrize("M", [16, 4096])
def test_outlier_and_precision_sweep(bits, F, M):
    """BASELINE config 4: K=N=8192, fp_features sweep, int4 and int8."""
    _check_sampled_rows(make_layer("sweep", M, 8192, 8192, bits, F=F, seed=3, device=dev(), clip=False), n_rows=24)
    torch.cuda.empty_cache()


def test_linearity_in_outlier_weights_full_size():
    """Size-independent property: scaling fp_weight by 2 changes the output by exactly the outlier product."""
    case = make_layer("lin", 2048, 4096, 4096, 4, F=256, seed=4, device=dev(), clip=False)
    base = case.module(case.x.unsqueeze(0))[0].float()
    fp_x = case.x[:, case.module.fp_indices]
    y = (fp_x.float() @ case.module.fp_weight.float().t())
    case.module.fp_weight.mul_(2)
    doubled = case.module(case.x.unsqueeze(0))[0].float()
    rms = base.pow(2).mean().sqrt()
    assert ((doubled - base) - y).abs().max() / rms < 2e-2
