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
