"""One Llama-2-style decoder block whose seven linear layers are MixedQLinear modules, wired the way the
reference wires them (QUIK experiments/llama.py:394-440): q/k/v share one quantized input (group of 3),
gate/up share one (group of 2), o and down quantize on their own (groups of 1); down_proj may run in 8 bits
(``int8_down_proj``).  Attention is plain torch (``F.scaled_dot_product_attention``) and rotary embedding one in-place pass over q and k
(``fused_rope``, bit-identical to the torch expression): they are the callers on either side of the hot path, not part of it.  The producers of the quantizers' inputs are fused into
the quantizer (``fused_producers``, default on): RMSNorm -> quantize for q/k/v and gate/up, SiLU(gate) * up -> quantize
for down_proj, each one pass over its input with the normalised / activated matrix never written to HBM.  Weights are random (seeded) and
quantized per output channel by symmetric round-to-nearest with clipping search, outlier columns are seed-chosen.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from ._lib import check, dtype_code, load, ptr, stream_of
from .qlinear import MixedQLinear, SharedQuantizedInput
from .workloads import rtn_clip_scales


class QuikLlamaBlock(torch.nn.Module):
    def __init__(self, hidden=4096, heads=32, intermediate=11008, kv_heads=None, bits=4, down_bits=8,
                 fp_features=256, seed=0, device="cuda", dtype=torch.float16, eps=1e-5, rope_theta=10000.0,
                 clip=True, keep_dense=False, fused_producers=True, fused_rope=True):
        super().__init__()
        kv_heads = kv_heads or heads
        self.hidden, self.heads, self.kv_heads, self.head_dim = hidden, heads, kv_heads, hidden // heads
        self.eps, self.rope_theta = eps, rope_theta
        g = torch.Generator().manual_seed(seed)
        kv_dim = self.head_dim * kv_heads
        # shared quantized inputs, in the reference's call order [k, v, q] and [up, gate]
        self.qkv_shared = SharedQuantizedInput(3)
        self.mlp_shared = SharedQuantizedInput(2)
        self.o_shared = SharedQuantizedInput(1)
        self.down_shared = SharedQuantizedInput(1)
        self.fused_producers = fused_producers
        self.fused_rope = fused_rope          # rotary embedding in one in-place pass (quik_rotary_inplace)
        self._rope_cache = {}
        dense = {}
        # the members of a group must agree on the outlier columns (the cached quantized input is shared):
        # each member draws them from a generator seeded per group
        mods = {}
        for name, out_f in (("k_proj", kv_dim), ("v_proj", kv_dim), ("q_proj", hidden)):
            perm_gen = torch.Generator().manual_seed(seed + 1)
            mods[name], dense[name] = self._member(hidden, out_f, bits, fp_features, perm_gen, g, device, dtype,
                                                   self.qkv_shared, clip)
        for name, out_f in (("up_proj", intermediate), ("gate_proj", intermediate)):
            perm_gen = torch.Generator().manual_seed(seed + 2)
            mods[name], dense[name] = self._member(hidden, out_f, bits, fp_features, perm_gen, g, device, dtype,
                                                   self.mlp_shared, clip)
        perm_gen = torch.Generator().manual_seed(seed + 3)
        mods["o_proj"], dense["o_proj"] = self._member(hidden, hidden, bits, fp_features, perm_gen, g, device, dtype,
                                                       self.o_shared, clip)
        perm_gen = torch.Generator().manual_seed(seed + 4)
        mods["down_proj"], dense["down_proj"] = self._member(intermediate, hidden, down_bits, fp_features, perm_gen, g,
                                                             device, dtype, self.down_shared, clip)
        for k, v in mods.items():
            setattr(self, k, v)
        self.dense = dense if keep_dense else None       # fake-quantized fp weights, for reference checks
        self.input_norm = torch.nn.Parameter(torch.ones(hidden, dtype=dtype, device=device), requires_grad=False)
        self.post_norm = torch.nn.Parameter(torch.ones(hidden, dtype=dtype, device=device), requires_grad=False)

    @staticmethod
    def _member(in_f, out_f, bits, fp_features, perm_gen, wgen, device, dtype, shared, clip):
        w = (0.02 * torch.randn(out_f, in_f, generator=wgen)).to(dtype).to(device)
        fp_idx = torch.sort(torch.randperm(in_f, generator=perm_gen)[:fp_features])[0] if fp_features > 0 else None
        mask = torch.ones(in_f, dtype=torch.bool)
        if fp_idx is not None:
            mask[fp_idx] = False
        int_cols = torch.arange(in_f)[mask].to(device)
        scales = rtn_clip_scales(w[:, int_cols], bits, clip=clip)
        lo, hi = (-8, 7) if bits == 4 else (-128, 127)
        w_rtn = w.clone()
        w_rtn[:, int_cols] = (scales * torch.clamp(torch.round(w[:, int_cols].float() / scales), lo, hi)).to(dtype)
        lin = torch.nn.Linear(in_f, out_f, bias=False)
        mod = MixedQLinear.from_float(lin, w_rtn, scales, shared_input=shared, fp_indices=fp_idx, bits=bits).to(device)
        return mod, w_rtn

    # ---- the non-linear glue (plain torch) ----------------------------------------------------
    def _rms_norm(self, x, weight):
        v = x.float()
        v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)
        return (v.to(x.dtype)) * weight

    def _angles(self, s, device, dtype):
        """cos / sin of the rotary angles for positions 0..s-1, [s, head_dim/2] in ``dtype`` (cached per length)."""
        key = (s, str(device), dtype)
        if self._rope_cache.get("key") != key:
            inv = 1.0 / (self.rope_theta ** (torch.arange(0, self.head_dim, 2, device=device).float() / self.head_dim))
            ang = torch.outer(torch.arange(s, device=device).float(), inv)
            self._rope_cache = {"key": key, "cos": ang.cos().to(dtype).contiguous(),
                                "sin": ang.sin().to(dtype).contiguous()}
        return self._rope_cache["cos"], self._rope_cache["sin"]

    def _rope(self, q, k):
        """q * cos + rotate_half(q) * sin on [b, heads, s, head_dim] views (plain torch)."""
        s = q.shape[-2]
        c, sn = self._angles(s, q.device, q.dtype)
        cos, sin = torch.cat([c, c], -1), torch.cat([sn, sn], -1)

        def rot(t):
            h = t.shape[-1] // 2
            return torch.cat([-t[..., h:], t[..., :h]], -1)
        return q * cos + rot(q) * sin, k * cos + rot(k) * sin

    def _rope_inplace(self, q, k, s):
        """The same rotation in one pass, in place on the q and k projections [s, heads*head_dim] (they are this
        block's own fresh outputs); bit-identical to ``_rope``."""
        c, sn = self._angles(s, q.device, q.dtype)
        with torch.cuda.device(q.device):
            check(load().quik_rotary_inplace(ptr(q), ptr(k), ptr(c), ptr(sn), dtype_code(q.dtype), s, self.heads,
                                             self.kv_heads, self.head_dim, stream_of(q)), "rotary")

    _fused_groups = None

    def fuse_groups(self, on=True):
        """Run each shared-input group (k/v/q and up/gate) as one layer with stacked weights: one quantizer call and
        one fused launch per group, same values per output column.  The member layers stay in place (state_dict,
        reference checks); the stacked copies cost their weights once more in HBM.  Off by default: at 2048 tokens the
        block measured 1.01 ms with stacked groups against 0.94 ms without (the consumers then read strided slices of
        the wide outputs), so it only pays where launches, not bytes, dominate."""
        if not on:
            self._fused_groups = None
            return self
        self._qkv_sizes = [self.k_proj.out_features, self.v_proj.out_features, self.q_proj.out_features]
        # plain attribute (not a registered submodule): the copies must not appear in the state_dict
        object.__setattr__(self, "_fused_groups", (MixedQLinear.concat([self.k_proj, self.v_proj, self.q_proj]),
                                                   MixedQLinear.concat([self.up_proj, self.gate_proj])))
        return self

    def forward(self, x, linear=None):
        """x: [1, S, hidden].  ``linear(name, x)`` may replace the quantized layers (reference checks)."""
        lin = linear or (lambda name, t: getattr(self, name)(t))
        b, s, _ = x.shape
        fused = linear is None and self._fused_groups is not None
        # producers fused into the quantizers: only with the quantized layers in place, their fused forward, and the
        # member-wise groups (the stacked copies have no shared input)
        prod = (linear is None and self.fused_producers and not fused
                and all(getattr(self, n).fused for n in ("k_proj", "up_proj", "down_proj")))
        if prod:
            self.k_proj.quantize_rmsnorm(x, self.input_norm, self.eps)      # fills the q/k/v group's shared input
            h = x                                                           # only its shape is used below
        else:
            h = self._rms_norm(x, self.input_norm)
        if fused:
            k, v, q = self._fused_groups[0](h).split(self._qkv_sizes, dim=-1)
        else:
            k = lin("k_proj", h)
            v = lin("v_proj", h)
            q = lin("q_proj", h)
        inplace = (self.fused_rope and linear is None and not fused and b == 1 and q.is_contiguous()
                   and k.is_contiguous() and self.head_dim % 16 == 0)
        if inplace:
            self._rope_inplace(q, k, s)
        q = q.view(b, s, self.heads, self.head_dim).transpose(1, 2)
        k = k.view(b, s, self.kv_heads, self.head_dim).transpose(1, 2)
        v = v.view(b, s, self.kv_heads, self.head_dim).transpose(1, 2)
        if not inplace:
            q, k = self._rope(q, k)
        if self.kv_heads != self.heads:
            rep = self.heads // self.kv_heads
            k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=1.0 / math.sqrt(self.head_dim))
        a = a.transpose(1, 2).reshape(b, s, self.hidden)
        x = x + lin("o_proj", a)
        if prod:
            self.up_proj.quantize_rmsnorm(x, self.post_norm, self.eps)
            h = x
        else:
            h = self._rms_norm(x, self.post_norm)
        if fused:
            up, gate = self._fused_groups[1](h).split(self.up_proj.out_features, dim=-1)
        else:
            up = lin("up_proj", h)
            gate = lin("gate_proj", h)
        if prod:
            self.down_proj.quantize_silu_mul(gate, up)
            x = x + lin("down_proj", gate)                                  # `gate` only gives the shape
        else:
            x = x + lin("down_proj", F.silu(gate) * up)
        return x
