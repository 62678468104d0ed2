"""Pin the CPU oracle against outputs of the reference's own Python (tests/golden)."""
import os

import pytest
import torch

from oracle import fakequant, kernel_path as kp

GOLD = torch.load(os.path.join(os.path.dirname(__file__), "golden", "reference_python.pt"), weights_only=False)


def test_pack_to_i4_matches_reference():
    g = GOLD["pack"]
    assert torch.equal(kp.pack_to_i4(g["vals"]), g["packed"])
    assert torch.equal(kp.two_compl(g["vals"], 4), g["two_compl"])
    assert torch.equal(kp.unpack_i4(g["packed"]), g["vals"])


@pytest.mark.parametrize("idx", range(len(GOLD["from_float"])))
def test_from_float_buffers_match_reference(idx):
    c = GOLD["from_float"][idx]
    buf = kp.from_float_buffers(c["weight"], c["scales"], c["fp_indices"], c["bits"], bias=c["bias"])
    ref = c["buffers"]
    for name in ("weights_scales", "int_weight", "reduced_w", "int_indices", "fp_indices"):
        assert torch.equal(buf[name], ref[name]), name
    if "fp_weight" in ref:
        assert torch.equal(buf["fp_weight"], ref["fp_weight"])
    assert (buf["bias"] is None) == c["bias_is_none"]
    if buf["bias"] is not None:
        assert torch.equal(buf["bias"], ref["bias"])


@pytest.mark.parametrize("idx", range(len(GOLD["fakequant"])))
def test_fakequant_port_matches_reference(idx):
    c = GOLD["fakequant"][idx]
    layer_probe = fakequant.FakeQuantLinear(torch.empty(0), c["act_scales"], c["nfp"], c["bits"])
    int_cols = layer_probe.q_idx
    scale = fakequant.weight_rtn_params(c["w"][:, int_cols], c["bits"], clip=True)
    assert torch.equal(scale, c["w_scale"])
    w_dq = c["w"].clone()
    w_dq[:, int_cols] = fakequant.weight_rtn_quantize(c["w"][:, int_cols], scale, c["bits"])
    assert torch.equal(w_dq, c["w_dq"])
    layer = fakequant.FakeQuantLinear(w_dq.half(), c["act_scales"], c["nfp"], c["bits"])
    with torch.no_grad():
        y = layer(c["x"])
    assert torch.equal(y, c["y"])
