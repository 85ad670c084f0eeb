"""minml_b200: a B200-native (sm_100a) drop-in for the CUDA backend of MaciejKozarzewski/minml, restricted to the
convolution / matrix-multiply inference path.

The product is the shared library libminml_b200.so and its C ABI (include/minml_b200.h).  This package holds the
build recipe, a ctypes binding, and a Python mirror of the reference's host-side interface for this path
(`backend`: the free functions of include/minml/core/math.hpp; `layers`: Conv2D / Dense / ... forward orchestration)
used by the tests and the benchmark.  Nothing here computes on the CPU: importing `backend` without the built
library raises.
"""
from . import _abi  # noqa: F401

__all__ = ["_abi", "backend", "layers"]
