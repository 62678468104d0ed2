"""GPU: the reference's own layer module, unmodified, on this repository's `quik` package.

The reference's experiments/qlinear.py (placed byte for byte under oracle/_ref/ by oracle/build_ref.py, where a
reference checkout was available at build time) does `import quik` and calls quik.asymmetric.quantize,
quik.matmul.int4Matmul / int8Matmul and quik.asymmetric.dequantize.  With this repository's alias package on the path
its MixedQLinear must build from the same float layer, hold the same buffers, and its forward -- the reference's
five-operator sequence -- must give what this repository's layer gives.
"""
import importlib.util
import os
import sys

import pytest
import torch

from oracle import build_ref
from quik_b200.qlinear import MixedQLinear, SharedQuantizedInput
from quik_b200.workloads import rtn_clip_scales
from tests.gpu_util import assert_device_clean, dev, rel_rms_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref_qlinear():
    path = build_ref.module_path()
    if not os.path.isfile(path):
        pytest.skip("the reference's qlinear.py was not available when oracle/_ref was built")
    import quik  # noqa: F401  -- this repository's drop-in package is what the reference module imports
    assert "quik_b200" in os.path.realpath(sys.modules["quik"].asymmetric.__file__)
    spec = importlib.util.spec_from_file_location("reference_qlinear", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _float_layer(K, N, F, bits, seed, bias):
    g = torch.Generator().manual_seed(seed)
    # the outlier columns depend on (seed, K) only, so that the members of a group agree on them
    fp_idx = torch.sort(torch.randperm(K, generator=torch.Generator().manual_seed(seed + 1))[:F])[0] if F else None
    w = (0.02 * torch.randn(N, K, generator=g)).half().to(dev())
    mask = torch.ones(K, dtype=torch.bool)
    if F:
        mask[fp_idx] = False
    cols = torch.arange(K)[mask].to(dev())
    scales = rtn_clip_scales(w[:, cols], bits, clip=False)
    lo, hi = (-8, 7) if bits == 4 else (-128, 127)
    w[:, cols] = (scales * torch.clamp(torch.round(w[:, cols].float() / scales), lo, hi)).half()
    lin = torch.nn.Linear(K, N, bias=bias)
    if bias:
        lin.bias.data = (0.1 * torch.randn(N, generator=g)).half()
    return lin, w, scales, fp_idx, g


@pytest.mark.parametrize("M,K,N,F,bits,bias", [(2048, 4096, 1024, 256, 4, False), (300, 1088, 520, 64, 8, True),
                                                (16, 4352, 512, 256, 4, False), (129, 2048, 264, 0, 4, True)])
def test_reference_module_runs_on_this_package(ref_qlinear, M, K, N, F, bits, bias):
    lin, w, scales, fp_idx, g = _float_layer(K, N, F, bits, seed=M + N, bias=bias)
    theirs = ref_qlinear.MixedQLinear.from_float(lin, w, scales, fp_indices=fp_idx, bits=bits).to(dev())
    ours = MixedQLinear.from_float(lin, w, scales, fp_indices=fp_idx, bits=bits).to(dev())
    # same buffers: names, dtypes, shapes and contents, one for one
    sd_t, sd_o = theirs.state_dict(), ours.state_dict()
    assert list(sd_t.keys()) == list(sd_o.keys())
    for k in sd_t:
        assert sd_t[k].dtype == sd_o[k].dtype and sd_t[k].shape == sd_o[k].shape, k
        assert torch.equal(sd_t[k], sd_o[k]), k
    x = torch.randn(1, M, K, generator=g)
    if F:
        x[..., fp_idx] *= 20
    x = x.half().to(dev())
    y_ref = theirs(x)                       # the reference's forward: five operators of this package
    y_fused = ours(x)                       # this repository's forward: quantizer + one fused kernel
    assert y_ref.shape == y_fused.shape == (1, M, N) and y_ref.dtype == torch.float16
    assert rel_rms_err(y_fused.cpu(), y_ref.cpu()) < 1e-2
    ours.fused = False                      # same operator sequence through this repository's module: last place
    y_unfused = ours(x)
    assert torch.equal(y_unfused, y_ref)
    # a state_dict written by one loads into the other
    ours.load_state_dict(sd_t)
    theirs.load_state_dict(sd_o)
    assert_device_clean()


def test_reference_shared_input_group_runs_on_this_package(ref_qlinear):
    """q/k/v share one quantized input in the reference (experiments/llama.py:402-411): its SharedQuantizedInput
    with three of its modules on this package's operators."""
    K, F = 1088, 64
    shared = ref_qlinear.SharedQuantizedInput(3)
    mods, outs = [], []
    g = None
    for i, N in enumerate((256, 256, 520)):
        lin, w, scales, fp_idx, g = _float_layer(K, N, F, 4, seed=7, bias=False)     # same outlier columns for the group
        mods.append((ref_qlinear.MixedQLinear.from_float(lin, w, scales, shared_input=shared, fp_indices=fp_idx, bits=4).to(dev()),
                     MixedQLinear.from_float(lin, w, scales, fp_indices=fp_idx, bits=4).to(dev()), fp_idx))
    x = torch.randn(1, 200, K, generator=torch.Generator().manual_seed(3))
    x[..., mods[0][2]] *= 20
    x = x.half().to(dev())
    for theirs, ours, _ in mods:
        y = theirs(x)
        assert rel_rms_err(ours(x).cpu(), y.cpu()) < 1e-2
    assert shared.qint_x is None and shared.cur_group_elem == 0          # the cache was dropped after the third member
    assert_device_clean()
