"""Drop-in alias: ``import quik`` resolves to the quik_b200 operators, so code written against the
reference package (``quik.asymmetric.quantize``, ``quik.matmul.int4Matmul``, ...) runs unchanged."""
from quik_b200 import asymmetric, matmul, symmetric  # noqa: F401
from quik_b200 import __version__  # noqa: F401
