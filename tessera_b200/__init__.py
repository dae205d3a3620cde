"""tessera_b200: B200-native kernels behind tessera's matmul and attention lowering rules.

The product is the C ABI in include/tessera_b200.h (tessera_b200/lib/libtessera_b200.so);
this package is the thin Python face the tests and benchmarks use: `ops` wraps each entry
point over torch device tensors, `rules` mirrors the reference's rule / launch-argument
registry, `runner` drives the C++ decode runner.
"""
from . import _lib  # noqa: F401  (raises when the shared library is missing)
from ._lib import TesseraError  # noqa: F401

__all__ = ["TesseraError"]
