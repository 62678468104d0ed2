"""ctypes binding of libquik_b200.so (the C ABI declared in include/quik_b200.h).

The library must be present: there is no CPU or eager fallback.  Build it with
``python -m quik_b200.build``.
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libquik_b200.so")

QUIK_OK = 0
F16, BF16 = 0, 1
CFG_GEMM_ENGINE, CFG_TILE_N, CFG_SMALL_M, CFG_CTA_PAIR, CFG_PDL, CFG_MMA_ISSUERS, CFG_L2_HINT = 1, 2, 3, 4, 5, 6, 7
CFG_STREAM_PRELOAD = 8
CFG_STREAM_RING = 9
ENGINE_AUTO, ENGINE_TCGEN05, ENGINE_MMA_SYNC, ENGINE_TCGEN05_TS = 0, 1, 2, 3
SMALL_M_MAX = 16       # most tokens of the mma.sync weight-streaming engines
STREAM_M_MAX = 128     # most tokens of the tcgen05 weight-streaming engine

_vp, _i, _sz, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_float

# name -> (restype, argtypes); mirrors include/quik_b200.h one to one
SIGNATURES = {
    "quik_version": (ctypes.c_char_p, []),
    "quik_strerror": (ctypes.c_char_p, [_i]),
    "quik_last_cuda_error": (ctypes.c_char_p, []),
    "quik_config_set": (_i, [_i, _i]),
    "quik_config_get": (_i, [_i]),
    "quik_device_status": (_i, [_i]),
    "quik_gemm_plan": (_i, [_i, _i, _i, _i, ctypes.POINTER(_i), ctypes.POINTER(_i)]),
    "quik_debug_counters": (_i, [_vp]),
    "quik_selftest_bounded_wait": (_i, [ctypes.c_uint, _vp, _vp]),
    "quik_asym_quantize": (_i, [_vp, _i, _i, _i, _vp, _i, _vp, _i, _i, _vp, _vp, _vp, _vp]),
    "quik_asym_quantize_u16": (_i, [_vp, _i, _i, _i, _vp, _i, _vp, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "quik_rmsnorm_quantize_u16": (_i, [_vp, _vp, _f, _i, _i, _i, _vp, _i, _vp, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "quik_silu_mul_quantize_u16": (_i, [_vp, _vp, _i, _i, _i, _vp, _i, _vp, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "quik_asym_find_meta": (_i, [_vp, _i, _i, _i, _i, _vp, _vp]),
    "quik_asym_quantize_old": (_i, [_vp, _i, _vp, _i, _i, _i, _vp, _vp]),
    "quik_asym_dequantize": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "quik_sym_quantize": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp]),
    "quik_sym_dequantize": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _i, _i, _vp]),
    "quik_int8_matmul": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "quik_int4_matmul_scratch_bytes": (_sz, [_i, _i, _i]),
    "quik_int4_matmul": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _sz, _vp]),
    "quik_int4_matmul_fixed_scratch": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "quik_unpack_int4": (_i, [_vp, _vp, _i, _i, _vp]),
    "quik_rotary_inplace": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "quik_copy_2d": (_i, [_vp, _sz, _vp, _sz, _sz, _sz, _vp]),
    "quik_copy_2d_sm": (_i, [_vp, _sz, _vp, _sz, _sz, _sz, _i, _vp]),
    "quik_fused_dequantize": (_i, [_vp, _vp, _i, _vp, _vp, _f, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _sz, _vp]),
    "quik_mixed_linear_ld": (_i, [_vp, _i, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, ctypes.c_longlong, _i, _i, _i, _i, _i, _i, _vp]),
    "quik_mixed_linear": (_i, [_vp, _i, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m quik_b200.build` "
                "(quik_b200 has no fallback path)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(status: int, what: str) -> None:
    """Turn a status code into the RuntimeError the reference would raise (TORCH_CHECK)."""
    if status != QUIK_OK:
        lib = load()
        msg = lib.quik_strerror(status).decode()
        detail = lib.quik_last_cuda_error().decode() if status == -6 else ""
        raise RuntimeError(f"{what}: {msg}" + (f" [{detail}]" if detail else ""))


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float16:
        return F16
    if dtype == torch.bfloat16:
        return BF16
    raise RuntimeError(f"expected a float16 or bfloat16 tensor, got {dtype}")


def ptr(t) -> int | None:
    return None if t is None or t.numel() == 0 else t.data_ptr()


def stream_of(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def require_cuda_contiguous(op: str, **tensors) -> None:
    """The reference's checkAllContiguous / checkDeviceType (e.g. src/asymmetric/asymmetric.cpp:19-23)."""
    dev = None
    for name, t in tensors.items():
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(f"{op}: expected tensor for argument '{name}' to be on a CUDA device")
        if not t.is_contiguous():
            raise RuntimeError(f"{op}: expected tensor for argument '{name}' to be contiguous")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"{op}: expected all tensors on the same GPU, got {dev} and {t.device}")


def set_engine(engine: int) -> None:
    check(load().quik_config_set(CFG_GEMM_ENGINE, engine), "quik_config_set")


def config_get(key: int) -> int:
    """Current value of a process-wide setting (the library's own word, not a Python-side copy)."""
    return load().quik_config_get(key)


def set_tile_n(n: int) -> None:
    check(load().quik_config_set(CFG_TILE_N, n), "quik_config_set")


def set_cta_pair(mode: int) -> None:
    """0 = CTA pairs when M > 128, 1 = never, 2 = always."""
    check(load().quik_config_set(CFG_CTA_PAIR, mode), "quik_config_set")


SMALL_M_OFF, SMALL_M_AUTO, SMALL_M_MMA_SYNC, SMALL_M_TCGEN05, SMALL_M_TMA_MMA = 0, 1, 2, 3, 4


def set_small_m(mode) -> None:
    """Engine for layers with at most SMALL_M_MAX tokens: 0 = none (tensor-core GEMM on widened weights),
    1 / True = weight streaming, engine by layer size, 2 = mma.sync fed by direct loads, 3 = tcgen05 fed by a TMA
    ring, 4 = mma.sync fed by a TMA ring."""
    check(load().quik_config_set(CFG_SMALL_M, int(mode)), "quik_config_set")


def set_mma_issuers(n: int) -> None:
    """1 or 2 threads issue the integer products of a tile (tcgen05 engine with both operands in shared memory)."""
    check(load().quik_config_set(CFG_MMA_ISSUERS, int(n)), "quik_config_set")


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch of the layer's kernels (default on); off = plain stream order."""
    check(load().quik_config_set(CFG_PDL, int(bool(on))), "quik_config_set")


def device_status(clear: bool = True) -> int:
    return load().quik_device_status(int(clear))
