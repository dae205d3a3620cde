"""tessera_b200: B200-native kernels behind tessera's matmul and attention lowering rules.

The product is the C ABI in include/tessera_b200.h (tessera_b200/lib/libtessera_b200.so);
this package is the thin Python face the tests and benchmarks use: `ops` wraps each entry
point over torch device tensors, `rules` mirrors the reference's rule / launch-argument
registry, `runner` drives the C++ decode runner.
"""
__all__ = ["TesseraError"]


def __getattr__(name):
    # The shared library is loaded on first use, not on import of the package, so that
    # `python -m tessera_b200.build` can run before the library exists.  Every module that does work
    # (`ops`, `runner`, ...) imports `_lib`, which raises when the library is missing: there is no
    # CPU path.
    if name == "TesseraError":
        from ._lib import TesseraError
        return TesseraError
    raise AttributeError(name)
