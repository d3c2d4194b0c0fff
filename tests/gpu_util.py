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
# From this many activation rows on, linears over fp16 / packed weights run as
# tensor-core GEMMs on fp16 copies of the activations, as the reference's cuBLAS path
# does (cuda/kernels.cu:600-633); csrc/gemm.cuh holds the same constant.
GEMM_MIN_ROWS = 32


def fp16_close(got, want, frac=4e-3):
    """Results of the tensor-core path against an fp32 computation: operands were
    rounded to fp16 (2^-11 relative each), so the error is bounded relative to the
    scale of the output, not element by element."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape
    scale = float(np.abs(want).max())
    err = float(np.abs(got - want).max())
    assert np.isfinite(got).all() and err <= frac * scale + 1e-6, f"max error {err:.3e} vs scale {scale:.3e}"


def close(got, want, rows, tol):
    """tol (an assert_allclose dict) below GEMM_MIN_ROWS rows, fp16_close from there on."""
    if rows >= GEMM_MIN_ROWS:
        fp16_close(got, want)
    else:
        np.testing.assert_allclose(got, want, **tol)
