"""quik.symmetric -- reference names and keyword arguments (QUIK src/symmetric/symmetric.cpp:108-186)."""
from __future__ import annotations

import torch

from ._lib import check, load, ptr, require_cuda_contiguous, stream_of
from .asymmetric import _fused

__all__ = ["quantize", "dequantize", "int4FusedDequantize", "int8FusedDequantize",
           "int4SpFusedDequantize", "int8SpFusedDequantize"]


def quantize(src, scale, bits):
    """symmetric.cpp:9-21: q = rn(src / scale[row]); bits=4 packs two nibbles per byte. fp16 only."""
    require_cuda_contiguous("quantize", src=src, scale=scale)
    if bits not in (4, 8):
        raise RuntimeError("Unsupported data type")
    if src.dtype != torch.float16 or scale.dtype != torch.float16:
        raise RuntimeError("quantize: expected float16 tensors")
    rows, cols = src.shape
    if scale.shape[0] != rows:
        raise RuntimeError(f"quantize: expected scale to have size {rows} at dimension 0")
    with torch.cuda.device(src.device):
        if bits == 4:
            dst = torch.empty((rows, (cols - 1) // 2 + 1), dtype=torch.uint8, device=src.device)
        else:
            dst = torch.empty((rows, cols), dtype=torch.int8, device=src.device)
        check(load().quik_sym_quantize(ptr(src), ptr(scale), rows, cols, bits, ptr(dst), stream_of(src)), "quantize")
    return dst


def dequantize(x, scale_row, scale_col, y, bits):
    """symmetric.cpp:23-42: out = half(x) * scale_row * scale_col + y in fp16 ops; bits = 8, 16 or 32
    names the type of x (int8, fp16, int32)."""
    require_cuda_contiguous("dequantize", x=x, scale_row=scale_row, scale_col=scale_col, y=y)
    want = {8: torch.int8, 16: torch.float16, 32: torch.int32}
    if bits not in want:
        raise RuntimeError("Unsupported data type")
    if x.dtype != want[bits]:
        raise RuntimeError(f"dequantize: x must be {want[bits]} for bits={bits}")
    rows, cols = x.shape
    if y.shape != x.shape:
        raise RuntimeError("dequantize: x and y must have the same size")
    if scale_row.shape[0] != rows or scale_col.numel() != cols:
        raise RuntimeError("dequantize: scale sizes do not match x")
    with torch.cuda.device(x.device):
        out = torch.empty_like(y)
        check(load().quik_sym_dequantize(ptr(x), bits, ptr(scale_row), ptr(scale_col), ptr(y), ptr(out), rows, cols,
                                         stream_of(x)), "dequantize")
    return out


def int4FusedDequantize(A, B, scale_row, scale_col, y):
    """symmetric.cpp:44-56 (fp32 arithmetic, one rounding)."""
    return _fused("int4FusedDequantize", 4, A, B, scale_row, scale_col, 0.0, None, None, y)


def int8FusedDequantize(A, B, scale_row, scale_col, y):
    """symmetric.cpp:58-70."""
    return _fused("int8FusedDequantize", 8, A, B, scale_row, scale_col, 0.0, None, None, y)


def int4SpFusedDequantize(*args, **kwargs):
    raise NotImplementedError("2:4 sparse kernels are outside the scope of quik_b200")


def int8SpFusedDequantize(*args, **kwargs):
    raise NotImplementedError("2:4 sparse kernels are outside the scope of quik_b200")
