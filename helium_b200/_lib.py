"""ctypes binding of libhelium_b200.so (the C ABI declared in include/helium_b200.h).

The shared library is the product.  If it has not been built, importing this module raises: there
is no Python or CPU fallback for any kernel.
"""
from __future__ import annotations

import ctypes as C
import os

from ._abi import HE_MAX_RANK, SIGNATURES, HeGraphDesc, HeNode  # noqa: F401  (re-exported)

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libhelium_b200.so")


class HeliumError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"helium_b200 status {status}: {message}")
        self.status = status
        self.message = message


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing. Build it with `python helium_b200/build.py` "
            "(nvcc, sm_100a). helium_b200 has no fallback path without its CUDA library.")
    lib = C.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = header and library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


lib = _load()


def check(status: int) -> None:
    if status != 0:
        raise HeliumError(status, lib.he_last_error_string().decode("utf-8", "replace"))
