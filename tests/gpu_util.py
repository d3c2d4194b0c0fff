"""Helpers for the GPU parity tests: device buffers (torch is only the allocator)
and the C-ABI binding."""
import importlib

import numpy as np
import torch

pkg = importlib.import_module("jdm-ghassan_v1_flach_b200")
ops = importlib.import_module("jdm-ghassan_v1_flach_b200.ops")
B200Error = pkg.B200Error


def dev(a):
    """numpy -> CUDA tensor holding the same bytes (uint16 travels as int16)."""
    if a is None:
        return None
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    return torch.from_numpy(a).cuda()


def host(t, dtype=None):
    a = t.detach().cpu().numpy()
    if dtype is not None:
        a = a.view(dtype)
    return a


def zeros(shape, dtype=torch.float32):
    return torch.zeros(shape, dtype=dtype, device="cuda")


def empty(shape, dtype=torch.float32):
    # poison instead of garbage so an unwritten output is caught
    t = torch.empty(shape, dtype=dtype, device="cuda")
    if dtype == torch.float32:
        t.fill_(float("nan"))
    else:
        t.fill_(-7)
    return t


def sync():
    torch.cuda.synchronize()


# Tolerances.  fp32 kernels that only differ from the oracle by summation order:
SUM_ORDER = dict(rtol=2e-4, atol=2e-5)
# The stated bound for activations/logits vs the reference CPU path:
ACTIVATION = dict(rtol=1e-2, atol=2e-2)
