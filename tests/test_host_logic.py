"""CPU-only: host-side logic of the layer (buffer schema, packing, workload generators)."""
import os

import pytest
import torch

from oracle import fakequant, kernel_path as kp
from quik_b200 import qlinear, workloads

GOLD = torch.load(os.path.join(os.path.dirname(__file__), "golden", "reference_python.pt"), weights_only=False)


def test_pack_to_i4_matches_reference_fixture():
    g = GOLD["pack"]
    assert torch.equal(qlinear.pack_to_i4(g["vals"]), g["packed"])
    assert torch.equal(qlinear.two_compl(g["vals"], 4), g["two_compl"])


@pytest.mark.parametrize("idx", range(len(GOLD["from_float"])))
def test_from_float_matches_reference_fixture(idx):
    if torch.cuda.is_available():
        pytest.skip("fixture comparison runs on CPU tensors")
    c = GOLD["from_float"][idx]
    lin = torch.nn.Linear(c["weight"].shape[1], c["weight"].shape[0], bias=c["bias"] is not None)
    if c["bias"] is not None:
        lin.bias.data = c["bias"]
    mod = qlinear.MixedQLinear.from_float(lin, c["weight"], c["scales"], fp_indices=c["fp_indices"], bits=c["bits"])
    got = dict(mod.named_buffers())
    assert set(got) == set(c["buffers"])
    for name, ref in c["buffers"].items():
        assert got[name].dtype == ref.dtype and got[name].shape == ref.shape, name
        assert torch.equal(got[name], ref), name
    assert (mod.bias is None) == c["bias_is_none"]


def test_constructor_buffer_schema():
    m = qlinear.MixedQLinear(64, 16, fp_features_num=8, bits=4)
    shapes = {k: (tuple(v.shape), v.dtype) for k, v in m.named_buffers()}
    assert shapes["weights_scales"] == ((16, 1), torch.float16)
    assert shapes["int_weight"] == ((16, 28), torch.uint8)
    assert shapes["bias"] == ((16,), torch.float16)
    assert shapes["int_indices"] == ((56,), torch.int64)
    assert shapes["fp_indices"] == ((8,), torch.int64)
    assert shapes["fp_weight"] == ((16, 8), torch.float16)
    assert shapes["reduced_w"] == ((1, 16), torch.float16)
    m8 = qlinear.MixedQLinear(64, 16, fp_features_num=0, bits=8, dtype=torch.bfloat16)
    assert m8.int_weight.dtype == torch.int8 and tuple(m8.int_weight.shape) == (16, 64)
    assert "fp_weight" not in dict(m8.named_buffers())
    ms = qlinear.MixedQLinear(64, 16, symm=True)
    assert "reduced_w" not in dict(ms.named_buffers())


def test_shared_quantized_input_protocol():
    s = qlinear.SharedQuantizedInput(2)
    s.qint_x = s.meta = s.fp_x = s.qscale_x = object()
    s.finish()
    assert s.qint_x is not None and s.cur_group_elem == 1
    s.finish()
    assert s.qint_x is None and s.meta is None and s.fp_x is None and s.qscale_x is None and s.cur_group_elem == 0


def test_u16_index_conversion():
    idx = torch.tensor([0, 1, 32767, 32768, 65535])
    u = qlinear._to_u16(idx)
    assert u.dtype == torch.int16
    assert [int(v) & 0xFFFF for v in u.tolist()] == idx.tolist()


@pytest.mark.parametrize("bits", [4, 8])
def test_rtn_clip_scales_match_oracle_port(bits):
    g = torch.Generator().manual_seed(bits)
    w = 0.02 * torch.randn(24, 96, generator=g)
    assert torch.allclose(workloads.rtn_clip_scales(w, bits), fakequant.weight_rtn_params(w, bits), rtol=0, atol=0)


def test_make_layer_on_cpu_is_consistent():
    if torch.cuda.is_available():
        pytest.skip("CPU-only construction check")
    c = workloads.make_layer("t", 8, 128, 32, 4, F=16, seed=0, device="cpu", keep_weight_dq=True)
    assert c.module.int_weight.shape == (32, 56) and c.fp_indices.numel() == 16
    assert torch.equal(torch.sort(c.fp_indices)[0], c.fp_indices)
    buf = kp.from_float_buffers(c.weight_dq, c.module.weights_scales.float(), c.fp_indices, 4)
    assert torch.equal(buf["int_indices"], c.module.int_indices)
    # tensor-parallel column shards are slices of the single-GPU layer
    full = workloads.make_layer("t", 8, 128, 32, 4, F=16, seed=0, device="cpu")
    half = workloads.make_layer("t", 8, 128, 32, 4, F=16, seed=0, device="cpu", n_slice=slice(16, 32))
    assert torch.equal(half.module.int_weight, full.module.int_weight[16:32])
    assert torch.equal(half.module.reduced_w, full.module.reduced_w[:, 16:32])
    assert torch.equal(half.x, full.x)
    assert c.ops == 2.0 * 8 * 32 * 128


def test_concat_stacks_member_layers():
    """MixedQLinear.concat: buffers of layers with the same column split stacked along the output dimension."""
    torch.manual_seed(0)
    K, F = 256, 32
    fp_idx = torch.randperm(K)[:F].sort()[0]
    mods = []
    for n in (64, 32, 96):
        lin = torch.nn.Linear(K, n, bias=False)
        w = (0.02 * torch.randn(n, K)).half()
        scales = w.float().abs().max(1, keepdim=True)[0] / 7
        mods.append(qlinear.MixedQLinear.from_float(lin, w, scales, fp_indices=fp_idx, bits=4))
    cat = qlinear.MixedQLinear.concat(mods)
    assert cat.out_features == 192 and cat.in_features == K and cat.fp_features_num == F
    assert torch.equal(cat.int_weight, torch.cat([m.int_weight for m in mods], 0))
    assert torch.equal(cat.weights_scales, torch.cat([m.weights_scales for m in mods], 0))
    assert torch.equal(cat.reduced_w, torch.cat([m.reduced_w for m in mods], 1))
    assert torch.equal(cat.fp_weight, torch.cat([m.fp_weight for m in mods], 0))
    assert torch.equal(cat.int_indices, mods[0].int_indices) and torch.equal(cat.fp_indices, mods[0].fp_indices)
    other = qlinear.MixedQLinear.from_float(torch.nn.Linear(K, 8, bias=False), (0.02 * torch.randn(8, K)).half(),
                                            torch.ones(8, 1), fp_indices=torch.arange(F), bits=4)
    with pytest.raises(AssertionError):
        qlinear.MixedQLinear.concat([mods[0], other])


def test_column_ids_are_range_checked():
    """The kernels trust their 16-bit column ids; the module refuses ids outside the row or overlapping sets."""
    import pytest
    from quik_b200.qlinear import MixedQLinear, _to_u16
    assert _to_u16(torch.tensor([0, 5, 65535])).tolist() == [0, 5, -1]
    with pytest.raises(RuntimeError):
        _to_u16(torch.tensor([0, 4096]), 4096)
    with pytest.raises(RuntimeError):
        _to_u16(torch.tensor([-1, 3]), 4096)
    m = MixedQLinear(64, 8, fp_features_num=8, bits=4)
    m.int_indices = torch.arange(56)
    m.fp_indices = torch.arange(56, 64)
    m._idx16()
    m2 = MixedQLinear(64, 8, fp_features_num=8, bits=4)
    m2.int_indices = torch.arange(56)
    m2.fp_indices = torch.arange(50, 58)            # overlaps the integer columns
    with pytest.raises(RuntimeError):
        m2._idx16()


def test_tp_row_blocks_cover_the_rows_once():
    """Row blocks of a tensor-parallel forward: disjoint, in order, covering [0, m), multiples of 256 rows except
    the last, one block for small outputs."""
    from quik_b200.tp import ColumnParallelMixedQLinear as CP
    lay = CP.__new__(CP)
    lay.world, lay.chunks = 4, None
    for m, width in [(4096, 28672), (4096, 2048), (16, 28672), (2048 + 128, 28672), (300, 1 << 20)]:
        blocks = lay._row_blocks(m, width)
        assert blocks[0][0] == 0 and blocks[-1][1] == m
        assert all(a[1] == b[0] for a, b in zip(blocks, blocks[1:]))
        assert all((r1 - r0) % 256 == 0 for r0, r1 in blocks[:-1])
        assert 1 <= len(blocks) <= CP.MAX_CHUNKS
    assert len(lay._row_blocks(4096, 2048)) == 1                   # 25 MB pulled: one block
    assert len(lay._row_blocks(4096, 28672)) == 4                  # 352 MB pulled
    lay.chunks = 2
    assert lay._row_blocks(4096, 2048) == [(0, 2048), (2048, 4096)]
    lay.chunks = 8
    assert len(lay._row_blocks(512, 2048)) == 2                    # never blocks of fewer than 256 rows


def test_diagnostics_and_bench_import_without_a_gpu():
    """The diagnostics module and bench.py import on a machine without a GPU (they fail only when asked to run)."""
    import importlib
    import subprocess
    import sys
    importlib.import_module("quik_b200.diagnostics")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--help"], capture_output=True, text=True)
    assert r.returncode == 0 and "--tp-copy" in r.stdout and "--stream-ring" in r.stdout
