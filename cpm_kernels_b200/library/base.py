"""Shared-library discovery and symbol binding.

Plays the role of cpm_kernels/library/base.py:41-96 (``Lib`` / ``Lib.bind``) for the one library this
package needs, with one deliberate difference: the reference defers a missing library to the first
call (its wrappers raise "Library ... is not initialized"); here a missing library or symbol raises
when the binding module is imported, because there is nothing to fall back to.
"""
from __future__ import annotations

import ctypes
import os
from typing import Callable, Sequence

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ENV_LIB = "CPMK_B200_LIB"


def find_library() -> str:
    """``$CPMK_B200_LIB`` if set, else the in-tree build ``cpm_kernels_b200/lib/libcpmk_b200.so``."""
    path = os.environ.get(ENV_LIB) or os.path.join(_PKG, "lib", "libcpmk_b200.so")
    if not os.path.exists(path):
        raise RuntimeError(
            "cpm_kernels_b200: CUDA library not found at %s. Build it with `python -m cpm_kernels_b200.build` "
            "(needs nvcc with sm_100a support). There is no CPU fallback." % path)
    return path


class Lib:
    def __init__(self, path: str | None = None):
        self.path = path or find_library()
        self._lib = ctypes.CDLL(self.path)

    def bind(self, name: str, arg_types: Sequence, ret_type) -> Callable:
        """Decorator in the style of the reference's ``Lib.bind``: the decorated function receives the
        bound C function through the attribute of the same name on this object."""
        try:
            func = getattr(self._lib, name)
        except AttributeError as e:
            raise RuntimeError("%s: undefined symbol: %s" % (self.path, name)) from e
        func.argtypes = list(arg_types)
        func.restype = ret_type
        setattr(self, name, func)

        def decorator(f):
            return f
        return decorator

    def has(self, name: str) -> bool:
        return hasattr(self._lib, name)
