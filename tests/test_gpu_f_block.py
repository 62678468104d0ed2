"""GPU: a Llama-2-style decoder block on MixedQLinear layers (BASELINE config 2, reduced and full width)."""
import pytest
import torch

from quik_b200.block import QuikLlamaBlock
from tests.gpu_util import assert_device_clean, dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("hidden,heads,inter,seq", [(512, 8, 1408, 96), (4096, 32, 11008, 256)])
def test_block_fused_matches_unfused_and_dense(hidden, heads, inter, seq):
    blk = QuikLlamaBlock(hidden, heads, inter, fp_features=64 if hidden < 4096 else 256, seed=0, device=dev(),
                         clip=False, keep_dense=True)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(1, seq, hidden, generator=g).half().to(dev())
    out = blk(x)
    assert out.shape == x.shape and torch.isfinite(out).all()
    # quantized-input caches are released after each group has been served
    assert blk.qkv_shared.qint_x is None and blk.qkv_shared.cur_group_elem == 0
    assert blk.mlp_shared.qint_x is None and blk.mlp_shared.cur_group_elem == 0
    # the reference's five-operator sequence on the same modules
    names = ["k_proj", "v_proj", "q_proj", "o_proj", "up_proj", "gate_proj", "down_proj"]
    for n in names:
        getattr(blk, n).fused = False
    unfused = blk(x)
    for n in names:
        getattr(blk, n).fused = True
    # Layer by layer the two paths agree to ~4e-6 of the RMS (tests/test_gpu_c_qlinear.py); inside a block the next
    # layer re-quantizes to 4 bits, so a value that sits on a rounding boundary can flip a code and move single
    # outputs by a fraction of a quantization step (1.1e-2 of the RMS after a 4096-wide block).  The check is
    # therefore on the RMS of the difference, with a loose cap on single elements.
    d = (out.float() - unfused.float())
    rms = unfused.float().pow(2).mean().sqrt()
    assert (d.pow(2).mean().sqrt() / rms).item() < 3e-2
    assert (d.abs().max() / rms).item() < 1.5
    # dense fp16 block with the same fake-quantized weights: differs only by the activation quantization error
    dense = blk(x, linear=lambda name, t: torch.nn.functional.linear(t, blk.dense[name]))
    # (a 4-bit code over a Gaussian row of 4096 values has a step of ~0.5 sigma, i.e. ~15% noise per layer on this
    # synthetic data; the bound only catches a wrong result, not a noisy one)
    rel = ((out.float() - dense.float()).pow(2).mean().sqrt() / dense.float().pow(2).mean().sqrt()).item()
    assert rel < 0.5, rel
    assert_device_clean()


@pytest.mark.parametrize("hidden,heads,inter,seq", [(512, 8, 1408, 96), (4096, 32, 11008, 16), (4096, 32, 11008, 256)])
def test_block_with_stacked_groups_matches_member_layers(hidden, heads, inter, seq):
    """k/v/q and up/gate as one layer each (MixedQLinear.concat): every output column is computed as in its member
    layer, so the block's output agrees with the member-wise block to the last place of a few elements at most."""
    blk = QuikLlamaBlock(hidden, heads, inter, fp_features=64 if hidden < 4096 else 256, seed=0, device=dev(), clip=False)
    x = torch.randn(1, seq, hidden, generator=torch.Generator().manual_seed(2)).half().to(dev())
    separate = blk(x).clone()
    # the stacked layers alone: identical columns
    h = blk._rms_norm(x, blk.input_norm)
    blk.fuse_groups(True)
    stacked = blk._fused_groups[0](h)[0]
    members = torch.cat([blk.k_proj(h)[0], blk.v_proj(h)[0], blk.q_proj(h)[0]], dim=-1)
    d = (stacked.float() - members.float()).abs().max() / members.float().pow(2).mean().sqrt()
    assert d.item() < 2e-3
    together = blk(x)
    rms = separate.float().pow(2).mean().sqrt()
    assert ((together.float() - separate.float()).pow(2).mean().sqrt() / rms).item() < 1e-2
    assert "_fused_groups" not in "".join(blk.state_dict().keys())
    blk.fuse_groups(False)
    assert torch.equal(blk(x), separate)
    assert_device_clean()
