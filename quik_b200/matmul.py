"""quik.matmul -- reference names (QUIK src/matmul/matmul.cpp:78-134).  Dense int4 / int8 GEMMs are
implemented; the 2:4-sparse and cuSPARSELt entry points raise NotImplementedError."""
from __future__ import annotations

import torch

from ._lib import check, load, ptr, require_cuda_contiguous, stream_of

__all__ = ["int4Matmul", "int8Matmul", "int4SpMatmul", "int8SpMatmul", "int4ReorderMeta", "int8ReorderMeta",
           "int4GenRandomSparseMeta", "int8GenRandomSparseMeta", "int4Uncompress", "int8Uncompress",
           "unpack_int4"]


def int4Matmul(A, B):
    """C = int4Matmul(A, B): A uint8 [M, K/2], B uint8 [N, K/2] packed int4 -> int32 [M, N]; matmul.cpp:8-13."""
    require_cuda_contiguous("int4Matmul", A=A, B=B)
    if A.dtype != torch.uint8 or B.dtype != torch.uint8:
        raise RuntimeError("int4Matmul: expected uint8 (packed int4) tensors")
    if A.shape[1] != B.shape[1]:
        raise RuntimeError("int4Matmul: A and B must have the same reduction size")
    M, N, K = A.shape[0], B.shape[0], A.shape[1] * 2
    with torch.cuda.device(A.device):
        C = torch.empty((M, N), dtype=torch.int32, device=A.device)
        nbytes = load().quik_int4_matmul_scratch_bytes(M, N, K)
        scratch = torch.empty((max(nbytes, 1),), dtype=torch.uint8, device=A.device)
        check(load().quik_int4_matmul(ptr(A), ptr(B), ptr(C), M, N, K, ptr(scratch), nbytes, stream_of(A)),
              "int4Matmul")
    return C


def int8Matmul(A, B):
    """C = int8Matmul(A, B): A int8 [M, K], B int8 [N, K] -> int32 [M, N]; matmul.cpp:43-48."""
    require_cuda_contiguous("int8Matmul", A=A, B=B)
    if A.dtype != torch.int8 or B.dtype != torch.int8:
        raise RuntimeError("int8Matmul: expected int8 tensors")
    if A.shape[1] != B.shape[1]:
        raise RuntimeError("int8Matmul: A and B must have the same reduction size")
    M, N, K = A.shape[0], B.shape[0], A.shape[1]
    with torch.cuda.device(A.device):
        C = torch.empty((M, N), dtype=torch.int32, device=A.device)
        check(load().quik_int8_matmul(ptr(A), ptr(B), ptr(C), M, N, K, stream_of(A)), "int8Matmul")
    return C


def unpack_int4(src):
    """Widen packed int4 [rows, K/2] (uint8) to int8 [rows, K]; low nibble first (include/int4.h:78-98)."""
    require_cuda_contiguous("unpack_int4", src=src)
    rows, cols = src.shape[0], src.shape[1] * 2
    with torch.cuda.device(src.device):
        dst = torch.empty((rows, cols), dtype=torch.int8, device=src.device)
        check(load().quik_unpack_int4(ptr(src), ptr(dst), rows, cols, stream_of(src)), "unpack_int4")
    return dst


def _sparse(*args, **kwargs):
    raise NotImplementedError("2:4 sparse kernels are outside the scope of quik_b200")


int4SpMatmul = int8SpMatmul = int4ReorderMeta = int8ReorderMeta = _sparse
int4GenRandomSparseMeta = int8GenRandomSparseMeta = int4Uncompress = int8Uncompress = _sparse
