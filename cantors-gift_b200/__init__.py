"""cg_b200: B200 (sm_100a) execution path for cantors-gift Executables.

The product is the C-ABI library lib/libcg_b200.so (sources under csrc/, declarations in
include/cg_b200.h). This package is the thin Python host layer over it: `capi` binds the
C ABI with ctypes, `ops` offers the same calls on torch CUDA tensors and on host buffers.
There is no CPU fallback anywhere in this package.
"""
from . import capi  # noqa: F401
from .capi import CgB200Error, lib, library_path  # noqa: F401
