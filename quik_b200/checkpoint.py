"""Loading the reference's quantized-model checkpoints into MixedQLinear modules.

The reference writes one dict with ``torch.save`` (QUIK experiments/llama.py:462-471): the float model's
``state_dict`` under ``"model"`` -- its linear weights already rounded to the quantization grid -- plus one entry
``"model.layers.<i>.<name>.scale"`` per quantized linear holding the per-output-channel weight scale (fp32
``[out_features, 1]``, experiments/llama.py:189).  ``llama_replace_with_kernels`` (experiments/llama.py:394-440) turns
it into layers: per decoder layer the groups ``[k, v, q]``, ``[o]``, ``[up, gate]``, ``[down]`` each share one
quantized input, the outlier columns of a linear are the ``fp_features`` largest entries of its activation scales
(``torch.sort(scales)[1][-fp_features:]``, experiments/llama.py:431-432; the scales come from a second file,
``act_scales/<model>.pt``, a dict ``"model.layers.<i>.<name>" -> fp32 [in_features]``), the bit width is the
activation quantizer's (8 for ``down_proj`` with ``--int8_down_proj``, experiments/llama.py:167,492).

This module does the same from the same two dicts, without the Hugging Face model object around them.
"""
from __future__ import annotations

import re
from collections import OrderedDict

import torch

from .qlinear import MixedQLinear, SharedQuantizedInput

# the reference's grouping and call order inside a decoder layer (experiments/llama.py:402-407)
LLAMA_GROUPS = (("self_attn.k_proj", "self_attn.v_proj", "self_attn.q_proj"), ("self_attn.o_proj",),
                ("mlp.up_proj", "mlp.gate_proj"), ("mlp.down_proj",))
_SCALE_KEY = re.compile(r"^model\.layers\.(\d+)\.(.+)\.scale$")


def checkpoint_layers(save_dict) -> list[int]:
    """Indices of the decoder layers that have quantized linears in the checkpoint."""
    return sorted({int(m.group(1)) for m in map(_SCALE_KEY.match, save_dict.keys()) if m})


def _fp_indices(act_scales, key, fp_features):
    if fp_features <= 0:
        return None
    if act_scales is None or key not in act_scales:
        raise KeyError(f"fp_features={fp_features} needs activation scales for '{key}'")
    return torch.sort(act_scales[key])[1][-fp_features:]      # experiments/llama.py:432


def load_quantized_layers(save_dict, act_scales=None, fp_features: int = 0, fp_features_frac: float | None = None,
                          bits: int = 4, int8_down_proj: bool = False, groups=LLAMA_GROUPS, device=None):
    """Builds the MixedQLinear modules of every decoder layer of a reference checkpoint.

    ``save_dict``: the loaded checkpoint (``{"model": state_dict, "model.layers.i.name.scale": ...}``).
    ``act_scales``: the loaded activation-scale dict, needed when outlier columns are kept.
    ``fp_features`` / ``fp_features_frac``: as the reference's ``--fp_features_num`` / ``--fp_features_frac``
    (experiments/llama.py:79-83: the larger of the count and the fraction of ``in_features``).
    Returns ``OrderedDict[layer index] -> OrderedDict[linear name] -> MixedQLinear`` with the members of a group
    sharing one ``SharedQuantizedInput`` in the reference's call order.  Linears without a scale entry are left out
    (the reference keeps them as float layers).
    """
    state = save_dict["model"]
    out = OrderedDict()
    for i in checkpoint_layers(save_dict):
        mods = OrderedDict()
        for group in groups:
            present = [n for n in group if f"model.layers.{i}.{n}.scale" in save_dict]
            shared = SharedQuantizedInput(len(present))
            for name in present:
                prefix = f"model.layers.{i}.{name}"
                weight = state[prefix + ".weight"]
                bias = state.get(prefix + ".bias")
                scale = save_dict[prefix + ".scale"]
                out_f, in_f = weight.shape
                lin = torch.nn.Linear(in_f, out_f, bias=bias is not None, device="meta")
                if bias is not None:
                    lin.bias = torch.nn.Parameter(bias.detach().clone(), requires_grad=False)
                nfp = fp_features
                if fp_features_frac is not None:
                    nfp = max(int(in_f * fp_features_frac), nfp)
                layer_bits = 8 if (int8_down_proj and name.endswith("down_proj")) else bits
                mod = MixedQLinear.from_float(lin, weight, scale.reshape(out_f, 1), shared_input=shared,
                                              fp_indices=_fp_indices(act_scales, prefix, nfp), bits=layer_bits)
                mods[name] = mod.to(device) if device is not None else mod
        out[i] = mods
    return out


def install_into(model_layers, quantized) -> None:
    """Swaps the linears of Hugging Face style decoder layers (``model.model.layers``) for the loaded modules, like
    ``modelutils.replace_single_mod_opt`` in the reference (experiments/modelutils.py:78-87)."""
    for i, mods in quantized.items():
        block = model_layers[i]
        for name, mod in mods.items():
            parent = block
            parts = name.split(".")
            for p in parts[:-1]:
                parent = getattr(parent, p)
            setattr(parent, parts[-1], mod)
