"""The reference's op names (`gai::ops::*` / `gai::cuda_ops::*`, core/ops.h:68-404,
cuda/cuda_ops.h) bound to the C ABI: `ops.linear_forward_q4(x, w, y, M, K, N, kind)`
calls `b200_linear_forward_q4` with the same argument order as the reference's
`cuda_ops::linear_forward_q4`.  Tensor arguments are torch CUDA tensors (or None).
"""
from .capi import lib

_RENAMED = {"copy": "b200_copy_f32"}   # cuda_ops::copy(float*, const float*, n)


def __getattr__(name):
    sym = _RENAMED.get(name, "b200_" + name)
    L = lib()
    if sym not in L.protos:
        raise AttributeError(f"no such op: {name}")
    return lambda *args: L.call(sym, *args)
