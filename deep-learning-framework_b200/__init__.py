"""B200-native matmul / Linear path of the KONAN AI engine, behind a C ABI.

The product is ``lib/libkai_b200.so`` (hand-written sm_100a CUDA; see ``csrc/``) and the
header ``include/kai_b200.h``.  This package is the Python binding used by the tests and the
benchmark: ``capi`` loads the library with ctypes and declares every entry point, and
``vmath`` mirrors the static methods of the reference's ``class VMath``
(source/engine/support/vmath.h) on top of it.

The directory name contains a hyphen, so import it with
``importlib.import_module("deep-learning-framework_b200")``.
"""
from . import capi  # noqa: F401
from . import vmath  # noqa: F401
from .capi import KaiError, load  # noqa: F401

__all__ = ["capi", "vmath", "KaiError", "load"]
