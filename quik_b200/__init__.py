"""quik_b200 -- B200 (sm_100a) implementation of QUIK's mixed-precision quantized linear layer.

``quik_b200.asymmetric``, ``quik_b200.matmul`` and ``quik_b200.symmetric`` carry the operator names
of the reference's ``quik`` package; ``quik_b200.qlinear`` carries ``MixedQLinear``.  All compute
runs in hand-written CUDA behind the C ABI of ``include/quik_b200.h`` (``libquik_b200.so``).
"""
from . import _lib  # noqa: F401
from . import asymmetric, matmul, symmetric  # noqa: F401

__version__ = "0.1.0"
__all__ = ["asymmetric", "matmul", "symmetric", "__version__"]
