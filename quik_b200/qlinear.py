"""MixedQLinear -- the mixed-precision quantized linear layer, API-compatible with the reference
module (QUIK experiments/qlinear.py:11-199): same constructor, ``from_float``, buffer names, dtypes
and shapes (so reference ``state_dict``s load), same ``SharedQuantizedInput`` protocol.

``forward`` runs two launches instead of the reference's five: the activation quantizer and one
fused kernel (integer GEMM + outlier fp16 GEMM + dequantize).  ``MixedQLinear.fused = False``
switches to the reference's own operator sequence (quantize -> int matmul -> F.linear ->
dequantize) on this package's operators.
"""
from __future__ import annotations

import numpy as np
import torch
from torch import Tensor

from . import _lib, asymmetric, matmul, symmetric
from ._lib import check, dtype_code, load, ptr, stream_of

__all__ = ["two_compl", "pack_to_i4", "SharedQuantizedInput", "MixedQLinear"]


def two_compl(x: Tensor, bits: int) -> Tensor:
    """Unsigned two's-complement representation of negative values (experiments/qlinear.py:11-12)."""
    return torch.where(x < 0, 2 ** bits + x, x)


def pack_to_i4(X: Tensor) -> Tensor:
    """Pack int4 values two per byte, even column in the low nibble (experiments/qlinear.py:15-18)."""
    X_i8 = two_compl(X.to(dtype=torch.int8), 4).to(torch.uint8)
    return X_i8[:, 0::2] | (X_i8[:, 1::2] << 4)


class SharedQuantizedInput:
    """Quantized-activation cache shared by the layers of one group (q/k/v, gate/up);
    experiments/qlinear.py:21-37.  The first member quantizes, the others reuse, and the cache is
    dropped after ``group_size`` calls to :meth:`finish`."""

    def __init__(self, group_size):
        self.qint_x = None
        self.fp_x = None
        self.qscale_x = None
        self.meta = None
        self.wide = False          # layout of qint_x: one code per byte (True) or the reference layout
        self.group_size = group_size
        self.cur_group_elem = 0

    def finish(self):
        self.cur_group_elem += 1
        if self.cur_group_elem == self.group_size:
            self.qint_x = None
            self.qscale_x = None
            self.meta = None
            self.fp_x = None
            self.cur_group_elem = 0


def _to_u16(idx: Tensor, cols: int | None = None) -> Tensor:
    """int64 column ids -> the same ids as 16-bit values (stored in an int16 tensor) on idx.device.

    The kernels index the row in shared memory with these ids without a range check (like the reference's kernels,
    src/asymmetric/asymmetric.cu:351-372), so ids outside [0, cols) are refused here, once per layer."""
    a64 = idx.detach().cpu().numpy().astype(np.int64)
    limit = 65536 if cols is None else cols
    if a64.size and (a64.min() < 0 or a64.max() >= limit):
        raise RuntimeError(f"MixedQLinear: column ids must lie in [0, {limit}), got [{a64.min()}, {a64.max()}]")
    return torch.from_numpy(a64.astype(np.uint16).view(np.int16).copy()).to(idx.device)


class MixedQLinear(torch.nn.Module):
    fused = True   # class-wide default; set on an instance to override
    # optional profiling hook: called as hook(module, begin: bool) right before / after the fused
    # GEMM launch (on the launching stream), e.g. to record CUDA events
    launch_hook = None
    # optional caller-owned output buffer [M, out_features] (e.g. symmetric memory of a tensor-parallel
    # group); used by the fused path when its shape, dtype and device match
    out_buffer = None

    def __init__(self, in_features, out_features, shared_input=None,
                 fp_features_num=0, symm=False, bits=4, dtype=torch.float16):
        super().__init__()
        self.fp_features_num = fp_features_num
        self.int_features_num = in_features - fp_features_num
        self.in_features = in_features
        self.out_features = out_features
        self.symmetric = symm
        self.bits = bits
        self.shared_input = shared_input
        self.dtype = dtype
        # buffer schema of experiments/qlinear.py:53-78
        self.register_buffer('weights_scales', torch.zeros((self.out_features, 1), dtype=self.dtype))
        if self.bits == 4:
            self.register_buffer('int_weight', torch.randint(1, 7, (self.out_features, self.int_features_num // 2),
                                                             dtype=torch.uint8))
        else:
            self.register_buffer('int_weight', torch.randint(-128, 127, (self.out_features, self.int_features_num),
                                                             dtype=torch.int8))
        self.register_buffer('bias', torch.zeros((self.out_features), dtype=dtype))
        self.register_buffer('int_indices', torch.zeros((self.int_features_num), dtype=torch.long))
        self.register_buffer('fp_indices', torch.zeros((self.fp_features_num), dtype=torch.long))
        if self.fp_features_num > 0:
            self.register_buffer('fp_weight', torch.randint(-8, 7, (self.out_features, self.fp_features_num)).to(dtype))
        if not self.symmetric:
            self.register_buffer('reduced_w', torch.zeros((1, self.out_features), dtype=dtype))
        self._cache = {}

    @classmethod
    def concat(cls, modules):
        """One layer whose output is the outputs of ``modules`` side by side.

        For layers that read the same input through the same column split (q/k/v, gate/up: a shared-input group of
        experiments/llama.py:402-411): per-channel scales, reduced_w, the integer and the outlier weights are simply
        stacked along the output dimension, so every output column is computed exactly as in its own layer, in one
        quantizer call and one fused launch instead of one launch per member."""
        m0 = modules[0]
        for m in modules[1:]:
            assert (m.bits, m.symmetric, m.in_features, m.fp_features_num, m.dtype) == \
                   (m0.bits, m0.symmetric, m0.in_features, m0.fp_features_num, m0.dtype), "layers differ in format"
            assert torch.equal(m.int_indices, m0.int_indices) and torch.equal(m.fp_indices, m0.fp_indices), \
                "layers differ in their outlier columns"
            assert (m.bias is None) == (m0.bias is None)
        out = cls(m0.in_features, sum(m.out_features for m in modules), fp_features_num=m0.fp_features_num,
                  symm=m0.symmetric, bits=m0.bits, dtype=m0.dtype)
        out.weights_scales = torch.cat([m.weights_scales for m in modules], 0)
        out.int_weight = torch.cat([m.int_weight for m in modules], 0).contiguous()
        out.bias = None if m0.bias is None else torch.cat([m.bias for m in modules], 0)
        out.int_indices, out.fp_indices = m0.int_indices, m0.fp_indices
        if m0.fp_features_num > 0:
            out.fp_weight = torch.cat([m.fp_weight for m in modules], 0).contiguous()
        if not m0.symmetric:
            out.reduced_w = torch.cat([m.reduced_w for m in modules], 1).contiguous()
        return out

    # ------------------------------------------------------------------ derived, lazily built operands
    def _cached(self, name, src: Tensor, make):
        key = (src.data_ptr(), src._version, str(src.device))
        ent = self._cache.get(name)
        if ent is None or ent[0] != key:
            ent = (key, make(src))
            self._cache[name] = ent
        return ent[1]

    def _idx16(self):
        k = self.in_features
        i16 = self._cached("int16", self.int_indices, lambda t: _to_u16(t, k))
        f16 = self._cached("fp16", self.fp_indices, lambda t: self._checked_fp_ids(t, k))
        return i16, f16

    def _checked_fp_ids(self, fp_idx, k):
        # integer and outlier columns must not overlap (experiments/qlinear.py:168-169 asserts the same at construction)
        both = torch.cat([self.int_indices.detach().cpu(), fp_idx.detach().cpu()])
        if both.numel() != k or torch.unique(both).numel() != k:
            raise RuntimeError("MixedQLinear: int_indices and fp_indices must together name every input column exactly once")
        return _to_u16(fp_idx, k)

    def _weight_codes_int8(self):
        """Weight codes one per byte, the operand layout of the tensor-core engine."""
        if self.bits == 8:
            return self.int_weight
        return self._cached("w8", self.int_weight, matmul.unpack_int4)

    def _operand_layouts(self, M):
        """(token codes packed?, weight codes packed?) for M tokens: which engine the fused launch will use."""
        small_m_mode = _lib.config_get(_lib.CFG_SMALL_M)
        row_ok = self.bits == 8 or self.int_features_num % 32 == 0
        stream = M <= _lib.STREAM_M_MAX and small_m_mode != _lib.SMALL_M_OFF and row_ok
        if self.bits == 8:
            return False, False
        if stream:
            return (M <= _lib.SMALL_M_MAX and small_m_mode != _lib.SMALL_M_TCGEN05), True
        return (row_ok and _lib.config_get(_lib.CFG_GEMM_ENGINE) == _lib.ENGINE_TCGEN05_TS), False

    def _fill_shared(self, quantized, wide):
        shared_input = self.shared_input
        if shared_input is None:
            raise RuntimeError("a fused producer needs a SharedQuantizedInput on the layer (group size >= 1)")
        shared_input.qint_x, shared_input.meta, shared_input.fp_x = quantized
        shared_input.wide = wide

    def quantize_rmsnorm(self, x, norm_weight, eps):
        """Quantizes RMSNorm(x) * norm_weight straight into this layer's shared input (one pass over x, the normalised
        activations never go to HBM).  The following forward calls of the group's members find the codes and skip their
        own quantizer; pass them any tensor of x's shape, dtype and device (it is not read)."""
        x2 = x[0] if x.dim() == 3 else x
        q_packed, _ = self._operand_layouts(x2.shape[0])
        i16, f16 = self._idx16()
        self._fill_shared(asymmetric.rmsnorm_quantize_u16(x2.contiguous(), norm_weight, eps, i16, f16, self.bits,
                                                          not q_packed), not q_packed)

    def quantize_silu_mul(self, gate, up):
        """Quantizes SiLU(gate) * up straight into this layer's shared input (see :meth:`quantize_rmsnorm`)."""
        g2 = gate[0] if gate.dim() == 3 else gate
        u2 = up[0] if up.dim() == 3 else up
        q_packed, _ = self._operand_layouts(g2.shape[0])
        i16, f16 = self._idx16()
        self._fill_shared(asymmetric.silu_mul_quantize_u16(g2.contiguous(), u2.contiguous(), i16, f16, self.bits,
                                                           not q_packed), not q_packed)

    # ------------------------------------------------------------------ forward
    def forward(self, x):
        if self.int_features_num <= 0:
            return torch.nn.functional.linear(x, self.fp_weight, self.bias)
        if torch.cuda.current_device() != x.device.index:
            torch.cuda.set_device(x.device)

        shared_input = self.shared_input
        if shared_input is None:
            shared_input = SharedQuantizedInput(1)
        if len(x.shape) == 3:
            x = x[0]
        if self.symmetric:
            return self._forward_symmetric(x, shared_input)
        if not self.fused:
            return self._forward_unfused(x, shared_input)

        M = x.shape[0]
        # Operand layouts by engine (the C side picks the engine from them, include/quik_b200.h):
        #   up to STREAM_M_MAX tokens: weight streaming, the weights stay in their storage format; the tcgen05
        #     streaming engine takes the token codes one per byte, the mma.sync engines (up to SMALL_M_MAX tokens, the
        #     default for 4-bit layers) packed like the weights;
        #   more tokens: tensor-core GEMM on weight codes one per byte; the quantizer writes the token codes one per
        #     byte too, except when the engine with the token operand in tensor memory is selected: it takes 4-bit
        #     token codes packed (the reference layout) and widens them on chip.
        # (a packed 4-bit row must be a multiple of 16 bytes for these engines; otherwise both operands one per byte)
        q_packed, w_packed = self._operand_layouts(M)
        wide = not q_packed
        if shared_input.qint_x is not None and self.bits == 4 and shared_input.wide != wide:
            raise RuntimeError("MixedQLinear: the shared quantized input was written in another code layout than this "
                               "member needs (the members of a group must run on the same engine)")
        if shared_input.qint_x is None:
            i16, f16 = self._idx16()
            shared_input.qint_x, shared_input.meta, shared_input.fp_x = asymmetric.quantize_u16(
                x, i16, f16, self.bits, wide)
            shared_input.wide = wide
        q = shared_input.qint_x
        w = self.int_weight if (w_packed or self.bits == 8) else self._weight_codes_int8()
        N = self.out_features
        hook = MixedQLinear.launch_hook
        with torch.cuda.device(x.device):
            ob = self.out_buffer
            if ob is not None and tuple(ob.shape) == (M, N) and ob.dtype == x.dtype and ob.device == x.device \
                    and ob.stride(1) == 1 and ob.stride(0) >= N:
                out = ob                         # may be a column range of a wider row-major matrix
            else:
                out = torch.empty((M, N), dtype=x.dtype, device=x.device)
            F = self.fp_features_num
            if hook is not None:
                hook(self, True)
            check(load().quik_mixed_linear_ld(
                ptr(q), int(q_packed), ptr(w), int(w_packed), ptr(shared_input.meta), ptr(self.weights_scales),
                ptr(self.reduced_w), ptr(shared_input.fp_x) if F > 0 else None,
                ptr(self.fp_weight) if F > 0 else None, ptr(self.bias) if self.bias is not None else None,
                ptr(out), out.stride(0), dtype_code(x.dtype), M, N, self.int_features_num, F, self.bits, stream_of(x)),
                "MixedQLinear.forward")
            if hook is not None:
                hook(self, False)
        shared_input.finish()
        return out.reshape((1, *out.shape))

    def _forward_unfused(self, x, shared_input):
        """The reference's operator sequence (experiments/qlinear.py:105-148)."""
        group_input = shared_input
        if shared_input.qint_x is not None and self.bits == 4 and shared_input.wide:
            # a fused member of the group left its codes one per byte; the reference operators take the packed layout
            shared_input = SharedQuantizedInput(1)
        if shared_input.qint_x is None:
            shared_input.qint_x, shared_input.meta, shared_input.fp_x = asymmetric.quantize(
                x, self.int_indices, self.fp_indices, self.bits)
            shared_input.wide = False
        if self.fp_features_num > 0:
            fp_result = torch.nn.functional.linear(shared_input.fp_x, self.fp_weight, self.bias)
        elif self.bias is not None:
            fp_result = self.bias.repeat(shared_input.qint_x.shape[0], 1)
        else:
            fp_result = torch.zeros((shared_input.qint_x.shape[0], self.out_features), dtype=x.dtype, device=x.device)
        if self.bits == 4:
            int_result = matmul.int4Matmul(shared_input.qint_x, self.int_weight)
        else:
            int_result = matmul.int8Matmul(shared_input.qint_x, self.int_weight)
        output = asymmetric.dequantize(int_result, shared_input.meta, self.weights_scales, self.reduced_w,
                                       fp_result, self.bits)
        shared_input.finish()
        if group_input is not shared_input:
            group_input.finish()
        return output.reshape((1, *output.shape))

    def _forward_symmetric(self, x, shared_input):
        """Symmetric-activation branch (experiments/qlinear.py:94-103,141-142).  The reference calls
        quik.symmetric.quantize / dequantize without their ``bits`` argument there, which raises
        TypeError against its own extension; this passes ``bits`` (and 32 for the int32 accumulator)."""
        if shared_input.qint_x is None:
            if self.fp_features_num > 0:
                int_x = x[:, self.int_indices].contiguous()
                shared_input.fp_x = x[:, self.fp_indices].contiguous()
            else:
                int_x = x
            reshaped_x = int_x.reshape((-1, int_x.shape[-1]))
            shared_input.qscale_x = (torch.max(torch.abs(reshaped_x), dim=1)[0].unsqueeze(1) / (
                    1 << (self.bits - 1) - 1)).to(torch.float16)
            shared_input.qint_x = symmetric.quantize(int_x, shared_input.qscale_x, self.bits)
        if self.fp_features_num > 0:
            fp_result = torch.nn.functional.linear(shared_input.fp_x, self.fp_weight, self.bias)
        elif self.bias is not None:
            fp_result = self.bias.repeat(shared_input.qint_x.shape[0], 1)
        else:
            fp_result = torch.zeros((shared_input.qint_x.shape[0], self.out_features), dtype=x.dtype, device=x.device)
        if self.bits == 4:
            int_result = matmul.int4Matmul(shared_input.qint_x, self.int_weight)
        else:
            int_result = matmul.int8Matmul(shared_input.qint_x, self.int_weight)
        output = symmetric.dequantize(int_result, shared_input.qscale_x, self.weights_scales.reshape(1, -1).contiguous(),
                                      fp_result, 32)
        shared_input.finish()
        return output.reshape((1, *output.shape))

    # ------------------------------------------------------------------ construction
    @staticmethod
    def from_float(module: torch.nn.Linear, weight_matrix, weights_scales, shared_input=None,
                   fp_indices=None, symm=False, bits=4):
        """Build the layer from a float ``nn.Linear`` (experiments/qlinear.py:150-199).

        ``weight_matrix`` holds the (already rounded-to-grid) weights, ``weights_scales`` the
        per-output-channel scale [out_features, 1].  Integer columns are stored as
        ``round(W / scale)`` (packed two per byte for 4 bits), outlier columns verbatim, and
        ``reduced_w`` is the fp32 row sum of the integer-column weights.
        """
        assert weights_scales.shape == (module.out_features, 1), 'weights_scales should have shape (out_features, 1)'
        assert weight_matrix.shape == (module.out_features, module.in_features)
        assert (symm and bits == 4) or not symm, "Symmetric quantization with 8 bits is not supported"
        int_indices = torch.arange(module.in_features)
        if fp_indices is None or len(fp_indices) == 0:
            fp_indices = torch.tensor([], dtype=int_indices.dtype)
        else:
            fp_indices = fp_indices.cpu()
            int_indices = int_indices[~torch.isin(int_indices, fp_indices)]
        assert torch.numel(int_indices) + torch.numel(fp_indices) == module.in_features, \
            'There are some duplication in the fp_indices!'

        int_module = MixedQLinear(module.in_features, module.out_features, shared_input,
                                  fp_features_num=torch.numel(fp_indices), symm=symm, bits=bits,
                                  dtype=weight_matrix.dtype)
        if torch.cuda.is_available():
            weight_matrix = weight_matrix.cuda()
        dev = weight_matrix.device
        int_module.weights_scales.copy_(weights_scales.to(weight_matrix.dtype))
        int_rounded_weight = (weight_matrix[:, int_indices.to(dev)] / weights_scales.to(dev)).round()
        if bits == 4:
            int_module.int_weight.copy_(pack_to_i4(int_rounded_weight.to(torch.int8)).cpu())
        else:
            int_module.int_weight.copy_(int_rounded_weight.to(torch.int8).cpu())
        if not symm:
            reduced_w = torch.sum(weight_matrix[:, int_indices.to(dev)].float(), dim=1, keepdim=True).to(
                weight_matrix.dtype)
            int_module.reduced_w.copy_(reduced_w.t().cpu())
        if module.bias is not None:
            int_module.bias.copy_(module.bias)
        else:
            int_module.bias = None
        int_module.int_indices.copy_(int_indices)
        int_module.fp_indices.copy_(fp_indices)
        if int_module.fp_features_num > 0:
            int_module.fp_weight.copy_(weight_matrix[:, fp_indices.to(dev)].to(weight_matrix.dtype))
        return int_module
