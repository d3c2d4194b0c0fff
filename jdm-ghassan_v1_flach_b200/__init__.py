"""B200-native backend for the quantized hybrid-layer forward step
(Mamba-2 + GQA + MoE) of the ghassan-ai engine.

The product is the C-ABI CUDA library `libb200ops.so` (sources in csrc/, ABI in
include/b200ops.h).  This package only binds it for the tests and the benchmark:

    capi   - ctypes binding generated from the header
    ops    - the reference's `gai::ops` function names over torch CUDA tensors
"""
from .capi import B200Error, Library, lib  # noqa: F401
