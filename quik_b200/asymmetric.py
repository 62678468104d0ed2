"""quik.asymmetric -- same names, keyword arguments and tensor layouts as the reference's
pybind submodule (QUIK src/asymmetric/asymmetric.cpp:134-245)."""
from __future__ import annotations

import torch

from . import _lib
from ._lib import check, dtype_code, load, ptr, require_cuda_contiguous, stream_of

__all__ = ["quantize", "quantizeOld", "dequantize", "find_meta", "int4FusedDequantize",
           "int8FusedDequantize", "int4SpFusedDequantize", "int8SpFusedDequantize", "quantize_u16"]


def _check_bits(bits):
    if bits not in (4, 8):
        raise RuntimeError("bits argument must be either 4 or 8")


def quantize(src, int_indices, fp_indices, bits):
    """(dst, meta, fp_x) = quantize(src, int_indices, fp_indices, bits); asymmetric.cpp:16-25."""
    require_cuda_contiguous("quantize", src=src)
    _check_bits(bits)
    if not int_indices.is_cuda or not fp_indices.is_cuda:
        raise RuntimeError("quantize: expected index tensors to be on a CUDA device")
    int_indices = int_indices.contiguous()
    fp_indices = fp_indices.contiguous()
    if int_indices.dtype != torch.int64 or fp_indices.dtype != torch.int64:
        raise RuntimeError("quantize: index tensors must be int64")
    rows, cols = src.shape
    num_int, num_fp = int_indices.numel(), fp_indices.numel()
    if num_fp + num_int != cols:
        raise RuntimeError("Quantize: number of fp and int columns is not equal to total number of columns")
    if num_int % 2 != 0:
        raise RuntimeError("Quantize: number of int columns has to be even (implementation detail)")
    with torch.cuda.device(src.device):
        if bits == 4:
            dst = torch.empty((rows, num_int // 2), dtype=torch.uint8, device=src.device)
        else:
            dst = torch.empty((rows, num_int), dtype=torch.int8, device=src.device)
        meta = torch.empty((2 * rows,), dtype=src.dtype, device=src.device)
        fp_x = torch.empty((rows, num_fp), dtype=src.dtype, device=src.device)
        check(load().quik_asym_quantize(ptr(src), dtype_code(src.dtype), rows, cols, ptr(int_indices), num_int,
                                        ptr(fp_indices), num_fp, bits, ptr(dst), ptr(meta), ptr(fp_x),
                                        stream_of(src)), "quantize")
    return dst, meta, fp_x


def quantize_u16(src, int_indices_u16, fp_indices_u16, bits, wide):
    """Layer-internal form of :func:`quantize`: 16-bit column ids (stored in int16 tensors) and an
    optional one-code-per-byte layout for 4-bit codes (the tensor-core GEMM operand)."""
    require_cuda_contiguous("quantize", src=src, int_indices=int_indices_u16, fp_indices=fp_indices_u16)
    _check_bits(bits)
    rows, cols = src.shape
    num_int, num_fp = int_indices_u16.numel(), fp_indices_u16.numel()
    with torch.cuda.device(src.device):
        if bits == 4 and not wide:
            dst = torch.empty((rows, num_int // 2), dtype=torch.uint8, device=src.device)
        else:
            dst = torch.empty((rows, num_int), dtype=torch.int8, device=src.device)
        meta = torch.empty((2 * rows,), dtype=src.dtype, device=src.device)
        fp_x = torch.empty((rows, num_fp), dtype=src.dtype, device=src.device)
        check(load().quik_asym_quantize_u16(ptr(src), dtype_code(src.dtype), rows, cols, ptr(int_indices_u16), num_int,
                                            ptr(fp_indices_u16), num_fp, bits, int(bool(wide)), ptr(dst), ptr(meta),
                                            ptr(fp_x), stream_of(src)), "quantize")
    return dst, meta, fp_x


def _alloc_quantized(src, num_int, num_fp, bits, wide):
    rows = src.shape[0]
    if bits == 4 and not wide:
        dst = torch.empty((rows, num_int // 2), dtype=torch.uint8, device=src.device)
    else:
        dst = torch.empty((rows, num_int), dtype=torch.int8, device=src.device)
    meta = torch.empty((2 * rows,), dtype=src.dtype, device=src.device)
    fp_x = torch.empty((rows, num_fp), dtype=src.dtype, device=src.device)
    return dst, meta, fp_x


def rmsnorm_quantize_u16(x, norm_weight, eps, int_indices_u16, fp_indices_u16, bits, wide):
    """quantize_u16(rmsnorm(x) * norm_weight) in one pass over ``x``: the normalised matrix is never written
    (LlamaRMSNorm arithmetic: fp32 statistics, rounded to x.dtype, times the weight in x.dtype)."""
    require_cuda_contiguous("rmsnorm_quantize", x=x, norm_weight=norm_weight, int_indices=int_indices_u16,
                            fp_indices=fp_indices_u16)
    _check_bits(bits)
    rows, cols = x.shape
    if norm_weight.numel() != cols or norm_weight.dtype != x.dtype:
        raise RuntimeError("rmsnorm_quantize: norm_weight must have one entry per column, of x's dtype")
    num_int, num_fp = int_indices_u16.numel(), fp_indices_u16.numel()
    with torch.cuda.device(x.device):
        dst, meta, fp_x = _alloc_quantized(x, num_int, num_fp, bits, wide)
        check(load().quik_rmsnorm_quantize_u16(ptr(x), ptr(norm_weight), float(eps), dtype_code(x.dtype), rows, cols,
                                               ptr(int_indices_u16), num_int, ptr(fp_indices_u16), num_fp, bits,
                                               int(bool(wide)), ptr(dst), ptr(meta), ptr(fp_x), stream_of(x)),
              "rmsnorm_quantize")
    return dst, meta, fp_x


def silu_mul_quantize_u16(gate, up, int_indices_u16, fp_indices_u16, bits, wide):
    """quantize_u16(silu(gate) * up) in one pass over ``gate`` and ``up``: the activated matrix is never written."""
    require_cuda_contiguous("silu_mul_quantize", gate=gate, up=up, int_indices=int_indices_u16, fp_indices=fp_indices_u16)
    _check_bits(bits)
    if gate.shape != up.shape or gate.dtype != up.dtype:
        raise RuntimeError("silu_mul_quantize: gate and up must have the same shape and dtype")
    rows, cols = gate.shape
    num_int, num_fp = int_indices_u16.numel(), fp_indices_u16.numel()
    with torch.cuda.device(gate.device):
        dst, meta, fp_x = _alloc_quantized(gate, num_int, num_fp, bits, wide)
        check(load().quik_silu_mul_quantize_u16(ptr(gate), ptr(up), dtype_code(gate.dtype), rows, cols,
                                                ptr(int_indices_u16), num_int, ptr(fp_indices_u16), num_fp, bits,
                                                int(bool(wide)), ptr(dst), ptr(meta), ptr(fp_x), stream_of(gate)),
              "silu_mul_quantize")
    return dst, meta, fp_x


def find_meta(src, bits):
    """meta = find_meta(src, bits); asymmetric.cpp:40-44 (flat [2*rows], (scale, zero) interleaved)."""
    if not src.is_cuda:
        raise RuntimeError("find_meta: expected tensor for argument 'src' to be on a CUDA device")
    _check_bits(bits)
    src = src.contiguous()
    rows, cols = src.shape
    with torch.cuda.device(src.device):
        meta = torch.empty((2 * rows,), dtype=src.dtype, device=src.device)
        check(load().quik_asym_find_meta(ptr(src), dtype_code(src.dtype), rows, cols, bits, ptr(meta),
                                         stream_of(src)), "find_meta")
    return meta


def quantizeOld(src, meta, bits):
    """dst = quantizeOld(src, meta, bits); asymmetric.cpp:8-14."""
    require_cuda_contiguous("quantize", src=src, meta=meta)
    _check_bits(bits)
    rows, cols = src.shape
    if meta.numel() != 2 * rows:
        raise RuntimeError(f"quantize: expected meta to have {2 * rows} elements, got {meta.numel()}")
    with torch.cuda.device(src.device):
        if bits == 4:
            dst = torch.empty((rows, (cols + 1) // 2), dtype=torch.uint8, device=src.device)
        else:
            dst = torch.empty((rows, cols), dtype=torch.int8, device=src.device)
        check(load().quik_asym_quantize_old(ptr(src), dtype_code(src.dtype), ptr(meta), rows, cols, bits, ptr(dst),
                                            stream_of(src)), "quantizeOld")
    return dst


def dequantize(x, meta, scale_col, wReduced, y, bits):
    """out = dequantize(x, meta, scale_col, wReduced, y, bits); asymmetric.cpp:27-38, asymmetric.cu:175-233."""
    require_cuda_contiguous("dequantize", x=x, meta=meta, scale_col=scale_col, y=y)
    _check_bits(bits)
    if not wReduced.is_cuda:
        raise RuntimeError("dequantize: expected tensor for argument 'wReduced' to be on a CUDA device")
    wReduced = wReduced.contiguous()
    if x.dtype != torch.int32:
        raise RuntimeError("dequantize: x must be int32")
    if x.numel() != y.numel():
        raise RuntimeError(f"Expected tensor for x to have same number of elements as tensor for y; but "
                           f"{x.numel()} does not equal {y.numel()} (while checking arguments for dequantize)")
    rows, cols = x.shape
    if meta.shape[0] != 2 * rows:
        raise RuntimeError(f"dequantize: expected meta to have size {2 * rows} at dimension 0")
    if scale_col.shape[0] != cols and scale_col.numel() != cols:
        raise RuntimeError(f"dequantize: expected scaleCol to have size {cols} at dimension 0")
    if wReduced.numel() != cols:
        raise RuntimeError(f"dequantize: expected wReduced to have size {cols} at dimension 1")
    if not (meta.dtype == scale_col.dtype == wReduced.dtype == y.dtype):
        raise RuntimeError("dequantize: meta, scale_col, wReduced and y must share one floating dtype")
    with torch.cuda.device(x.device):
        out = torch.empty_like(y)
        check(load().quik_asym_dequantize(ptr(x), ptr(meta), ptr(scale_col), ptr(wReduced), ptr(y), ptr(out),
                                          dtype_code(y.dtype), rows, cols, bits, stream_of(x)), "dequantize")
    return out


def _fused(op, bits, A, B, scale_row, scale_col, shift_value, zero_row, w_reduced, y):
    require_cuda_contiguous(op, A=A, B=B, scale_row=scale_row, scale_col=scale_col, zero_row=zero_row,
                            w_reduced=w_reduced, y=y)
    for name, t in (("scale_row", scale_row), ("scale_col", scale_col), ("zero_row", zero_row),
                    ("w_reduced", w_reduced), ("y", y)):
        if t is not None and t.dtype != torch.float16:
            raise RuntimeError(f"{op}: {name} must be float16")
    M, N = A.shape[0], B.shape[0]
    K = A.shape[1] * (2 if bits == 4 else 1)
    if B.shape[1] != A.shape[1]:
        raise RuntimeError(f"{op}: A and B must have the same reduction size")
    if scale_row.numel() != M or scale_col.numel() != N or y.shape != (M, N):
        raise RuntimeError(f"{op}: scale_row / scale_col / y do not match A and B")
    with torch.cuda.device(A.device):
        out = torch.empty((M, N), dtype=torch.float16, device=A.device)
        scratch, nbytes = None, 0
        if bits == 4:
            nbytes = load().quik_int4_matmul_scratch_bytes(M, N, K)
            scratch = torch.empty((max(nbytes, 1),), dtype=torch.uint8, device=A.device)
        check(load().quik_fused_dequantize(ptr(A), ptr(B), bits, ptr(scale_row), ptr(scale_col), float(shift_value),
                                           ptr(zero_row), ptr(w_reduced), ptr(y), ptr(out), M, N, K,
                                           ptr(scratch), nbytes, stream_of(A)), op)
    return out


def int4FusedDequantize(A, B, scale_row, scale_col, shift_value, zero_row, w_reduced, y):
    """asymmetric.cpp:46-66.  The arithmetic is done in fp32 with one final rounding (the reference
    rounds every operation to fp16 and can overflow for |acc| > 65504)."""
    return _fused("int4FusedDequantize", 4, A, B, scale_row, scale_col, shift_value, zero_row, w_reduced, y)


def int8FusedDequantize(A, B, scale_row, scale_col, shift_value, zero_row, w_reduced, y):
    """asymmetric.cpp:68-88."""
    return _fused("int8FusedDequantize", 8, A, B, scale_row, scale_col, shift_value, zero_row, w_reduced, y)


def int4SpFusedDequantize(*args, **kwargs):
    raise NotImplementedError("2:4 sparse kernels are outside the scope of quik_b200")


def int8SpFusedDequantize(*args, **kwargs):
    raise NotImplementedError("2:4 sparse kernels are outside the scope of quik_b200")
