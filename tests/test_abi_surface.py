"""CPU-only: the C-ABI library loads, exports every symbol the header declares, and the host-only
entry points behave; the Python surface carries the reference's operator names."""
import ctypes
import inspect
import os
import re

import pytest
import torch

from quik_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "quik_b200.h")


def _declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(quik_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = _declared_symbols()
    assert len(names) >= 19
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/quik_b200.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), set(names) ^ set(_lib.SIGNATURES)


def test_host_only_entry_points():
    lib = _lib.load()
    assert b"sm_100a" in lib.quik_version()
    assert lib.quik_strerror(0) == b"ok"
    assert b"4 or 8" in lib.quik_strerror(-2)
    assert lib.quik_int4_matmul_scratch_bytes(128, 256, 512) == 128 * 512 + 256 * 512
    assert lib.quik_int4_matmul_scratch_bytes(3, 5, 32) == 256 + 256
    assert lib.quik_config_set(_lib.CFG_GEMM_ENGINE, _lib.ENGINE_MMA_SYNC) == 0
    assert lib.quik_config_get(_lib.CFG_GEMM_ENGINE) == _lib.ENGINE_MMA_SYNC
    assert lib.quik_config_set(_lib.CFG_GEMM_ENGINE, 0) == 0
    assert lib.quik_config_set(_lib.CFG_GEMM_ENGINE, 9) != 0
    assert lib.quik_config_set(_lib.CFG_TILE_N, 192) == 0          # any multiple of 16 from 32 to 256
    assert lib.quik_config_get(_lib.CFG_TILE_N) == 192
    assert lib.quik_config_set(_lib.CFG_TILE_N, 200) != 0 and lib.quik_config_set(_lib.CFG_TILE_N, 272) != 0
    assert lib.quik_config_set(_lib.CFG_TILE_N, 0) == 0
    # argument validation happens before any CUDA call
    assert lib.quik_asym_quantize(None, 0, 4, 64, None, 56, None, 8, 3, None, None, None, None) == -2
    assert lib.quik_asym_quantize(None, 0, 4, 64, None, 55, None, 8, 4, None, None, None, None) == -3
    assert lib.quik_asym_quantize(None, 0, 4, 64, None, 56, None, 8, 4, None, None, None, None) == -1
    assert lib.quik_asym_quantize(None, 7, 4, 64, None, 56, None, 8, 4, None, None, None, None) == -5
    assert lib.quik_int8_matmul(None, None, None, 4, 4, 24, None) == -3
    assert lib.quik_int8_matmul(None, None, None, 4, 4, 32, None) == -1
    assert lib.quik_int4_matmul(1024, 2048, 4096, 4, 4, 64, None, 0, None) == -7
    # settings of the streaming engines: ranges checked, defaults restored
    for key, default, bad in ((_lib.CFG_STREAM_PRELOAD, 1, 3), (_lib.CFG_STREAM_RING, 2, 3), (_lib.CFG_MMA_ISSUERS, 1, 3)):
        assert lib.quik_config_get(key) == default
        assert lib.quik_config_set(key, bad) != 0 and lib.quik_config_get(key) == default
        other = 2 if key == _lib.CFG_MMA_ISSUERS else 0
        assert lib.quik_config_set(key, other) == 0 and lib.quik_config_get(key) == other
        assert lib.quik_config_set(key, default) == 0
    # rotary embedding and the copy kernel: shapes and alignment are refused before any CUDA call
    assert lib.quik_rotary_inplace(16, 16, 16, 16, 0, 4, 2, 2, 24, None) == -3          # head_dim % 16
    assert lib.quik_rotary_inplace(16, 16, 16, 16, 9, 4, 2, 2, 32, None) == -5          # dtype code
    assert lib.quik_rotary_inplace(None, None, None, None, 0, 0, 2, 2, 32, None) == 0   # no tokens: nothing to do
    assert lib.quik_rotary_inplace(16, 16, 16, 24, 0, 4, 2, 2, 32, None) == -4          # table not 16-byte aligned
    assert lib.quik_copy_2d_sm(16, 64, 32, 64, 24, 4, 0, None) == -4                    # width % 16
    assert lib.quik_copy_2d_sm(16, 16, 32, 64, 32, 4, 0, None) == -3                    # pitch below the width
    assert lib.quik_copy_2d_sm(None, 64, None, 64, 0, 4, 0, None) == 0                  # empty copy


def test_python_surface_matches_reference_names():
    import quik
    # QUIK src/asymmetric/asymmetric.cpp:134-245, src/matmul/matmul.cpp:78-134, src/symmetric/symmetric.cpp:108-186
    want = {
        quik.asymmetric: {"quantizeOld": ["src", "meta", "bits"],
                          "quantize": ["src", "int_indices", "fp_indices", "bits"],
                          "dequantize": ["x", "meta", "scale_col", "wReduced", "y", "bits"],
                          "find_meta": ["src", "bits"],
                          "int4FusedDequantize": ["A", "B", "scale_row", "scale_col", "shift_value", "zero_row", "w_reduced", "y"],
                          "int8FusedDequantize": ["A", "B", "scale_row", "scale_col", "shift_value", "zero_row", "w_reduced", "y"]},
        quik.matmul: {"int4Matmul": ["A", "B"], "int8Matmul": ["A", "B"]},
        quik.symmetric: {"quantize": ["src", "scale", "bits"],
                         "dequantize": ["x", "scale_row", "scale_col", "y", "bits"],
                         "int4FusedDequantize": ["A", "B", "scale_row", "scale_col", "y"],
                         "int8FusedDequantize": ["A", "B", "scale_row", "scale_col", "y"]},
    }
    for mod, fns in want.items():
        for name, params in fns.items():
            assert list(inspect.signature(getattr(mod, name)).parameters) == params, name
    for name in ("int4SpMatmul", "int8SpMatmul", "int4ReorderMeta", "int8ReorderMeta", "int4GenRandomSparseMeta",
                 "int8GenRandomSparseMeta", "int4Uncompress", "int8Uncompress"):
        with pytest.raises(NotImplementedError):
            getattr(quik.matmul, name)()


def test_ops_fail_loudly_without_a_gpu():
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    import quik
    x = torch.randn(4, 64).half()
    with pytest.raises(RuntimeError):
        quik.asymmetric.quantize(x, torch.arange(56), torch.arange(56, 64), 4)
    with pytest.raises(RuntimeError):
        quik.matmul.int8Matmul(torch.zeros(4, 16, dtype=torch.int8), torch.zeros(4, 16, dtype=torch.int8))
