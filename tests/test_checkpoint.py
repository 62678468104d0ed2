"""CPU: a checkpoint in the reference's layout (experiments/llama.py:462-476) loads into MixedQLinear modules that are
identical to modules built directly with from_float, grouped like experiments/llama.py:402-411."""
import io

import torch

from quik_b200 import checkpoint
from quik_b200.qlinear import MixedQLinear
from quik_b200.workloads import rtn_clip_scales

NAMES = {"self_attn.q_proj": (64, 64), "self_attn.k_proj": (32, 64), "self_attn.v_proj": (32, 64), "self_attn.o_proj": (64, 64),
         "mlp.gate_proj": (96, 64), "mlp.up_proj": (96, 64), "mlp.down_proj": (64, 96)}


def _reference_style_checkpoint(n_layers=2, seed=0):
    """What the reference's script writes: the float state_dict with weights on the grid, one scale per linear."""
    g = torch.Generator().manual_seed(seed)
    state, save, act = {}, {}, {}
    for i in range(n_layers):
        for name, (out_f, in_f) in NAMES.items():
            bits = 8 if name.endswith("down_proj") else 4
            w = (0.05 * torch.randn(out_f, in_f, generator=g)).half()
            scale = rtn_clip_scales(w, bits, clip=False)                       # fp32 [out, 1]
            lo, hi = (-8, 7) if bits == 4 else (-128, 127)
            state[f"model.layers.{i}.{name}.weight"] = (scale * torch.clamp(torch.round(w.float() / scale), lo, hi)).half()
            save[f"model.layers.{i}.{name}.scale"] = scale.float()
            act[f"model.layers.{i}.{name}"] = torch.rand(in_f, generator=g)
        state[f"model.layers.{i}.input_layernorm.weight"] = torch.ones(64).half()
    state["model.embed_tokens.weight"] = torch.zeros(10, 64).half()
    save["model"] = state
    return save, act


def test_reference_checkpoint_round_trip():
    save, act = _reference_style_checkpoint()
    buf = io.BytesIO()
    torch.save(save, buf)                                   # the reference's torch.save / torch.load
    buf.seek(0)
    loaded = torch.load(buf)
    assert checkpoint.checkpoint_layers(loaded) == [0, 1]
    layers = checkpoint.load_quantized_layers(loaded, act_scales=act, fp_features=8, bits=4, int8_down_proj=True)
    assert list(layers.keys()) == [0, 1]
    for i, mods in layers.items():
        assert set(mods.keys()) == set(NAMES)
        # groups share one quantized input of the right size, in the reference's call order
        qkv = [mods[n].shared_input for n in ("self_attn.k_proj", "self_attn.v_proj", "self_attn.q_proj")]
        assert qkv[0] is qkv[1] is qkv[2] and qkv[0].group_size == 3
        assert mods["mlp.up_proj"].shared_input is mods["mlp.gate_proj"].shared_input
        assert mods["mlp.up_proj"].shared_input.group_size == 2
        assert mods["self_attn.o_proj"].shared_input.group_size == 1
        assert mods["self_attn.o_proj"].shared_input is not mods["mlp.down_proj"].shared_input
        assert list(mods.keys())[:3] == ["self_attn.k_proj", "self_attn.v_proj", "self_attn.q_proj"]
        for name, mod in mods.items():
            out_f, in_f = NAMES[name]
            bits = 8 if name.endswith("down_proj") else 4
            assert mod.bits == bits and mod.fp_features_num == 8 and mod.bias is None
            prefix = f"model.layers.{i}.{name}"
            fp_idx = torch.sort(act[prefix])[1][-8:]
            direct = MixedQLinear.from_float(torch.nn.Linear(in_f, out_f, bias=False), save["model"][prefix + ".weight"],
                                             save[prefix + ".scale"], fp_indices=fp_idx, bits=bits)
            a, b = mod.state_dict(), direct.state_dict()
            assert list(a.keys()) == list(b.keys())
            for k in a:
                assert torch.equal(a[k].cpu(), b[k].cpu()), (name, k)


def test_checkpoint_without_outliers_and_with_fraction():
    save, act = _reference_style_checkpoint(n_layers=1)
    plain = checkpoint.load_quantized_layers(save, bits=4)
    assert all(m.fp_features_num == 0 for m in plain[0].values())
    frac = checkpoint.load_quantized_layers(save, act_scales=act, fp_features=4, fp_features_frac=0.125, bits=4)
    assert frac[0]["mlp.down_proj"].fp_features_num == 12 and frac[0]["self_attn.q_proj"].fp_features_num == 8


def test_install_into_replaces_linears():
    save, act = _reference_style_checkpoint(n_layers=1)
    layers = checkpoint.load_quantized_layers(save, bits=4)

    class Holder(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.self_attn = torch.nn.Module()
            self.mlp = torch.nn.Module()
            for name, (o, i) in NAMES.items():
                parent, leaf = name.split(".")
                setattr(getattr(self, parent), leaf, torch.nn.Linear(i, o, bias=False))

    blocks = [Holder()]
    checkpoint.install_into(blocks, layers)
    assert all(isinstance(getattr(getattr(blocks[0], n.split(".")[0]), n.split(".")[1]), MixedQLinear) for n in NAMES)
