"""Decode attention without device allocation (b200_attention_decode_ring_fp16_noalloc).

Who needs it: a host application that owns all device memory through its own pool, or
that cannot accept the device-wide synchronisation a cudaMalloc / cudaFree implies in
the middle of decoding.  The entry point keeps its split-KV partial results in an
array compiled into the library instead of the growing workspace.  Checked here
through the C ABI against the allocating entry point, on two consecutive calls with
different inputs and lengths (the built-in array keeps the first call's contents when
the second runs), plus the size limit.

This file sorts last on purpose: a run that stops at the first failure has then
already executed every other test.  It also passes when run alone in a fresh process.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = dict(rtol=2e-4, atol=2e-5)      # the tolerance of tests/test_gpu_attention.py


def _case(seed, H, KV, hd, cache_max):
    r = np.random.default_rng(seed)
    q = r.standard_normal((H, hd)).astype(np.float32)
    kc = r.standard_normal((cache_max, KV * hd)).astype(np.float16).view(np.uint16)
    vc = r.standard_normal((cache_max, KV * hd)).astype(np.float16).view(np.uint16)
    return q, kc, vc


def test_noalloc_matches_allocating_entry_point_twice_in_a_row():
    from gpu_util import dev, empty, host, ops
    H, KV, hd, cache_max = 12, 4, 128, 4096
    free_before = torch.cuda.mem_get_info()[0]
    # (seed, ring_start, pinned, cur_len, window): a long context first, then a short one, so
    # the second call sees a scratch array still full of the first call's partial results
    for seed, rs, pin, cur, win in ((1, 0, 0, 4096, 0), (2, 100, 8, 777, 0), (3, 0, 0, 1, 0), (4, 0, 0, 900, 128)):
        q, kc, vc = _case(seed, H, KV, hd, cache_max)
        dq, dk, dv = dev(q), dev(kc), dev(vc)
        want, got = empty((H, hd)), empty((H, hd))
        ops.attention_decode_ring_fp16(dq, dk, dv, want, H, KV, hd, rs, pin, cur, cache_max, hd ** -0.5, None, win)
        ops.attention_decode_ring_fp16_noalloc(dq, dk, dv, got, H, KV, hd, rs, pin, cur, cache_max, hd ** -0.5, win)
        np.testing.assert_allclose(host(got), host(want), **TOL)
    assert np.isfinite(host(got)).all()
    assert torch.cuda.mem_get_info()[0] <= free_before          # sanity: nothing was freed behind our back


def test_noalloc_other_shapes_and_limit():
    from gpu_util import B200Error, dev, empty, host, ops
    for H, KV, hd in ((32, 8, 128), (4, 4, 32), (16, 1, 64)):
        q, kc, vc = _case(H + hd, H, KV, hd, 600)
        want, got = empty((H, hd)), empty((H, hd))
        ops.attention_decode_ring_fp16(dev(q), dev(kc), dev(vc), want, H, KV, hd, 0, 0, 600, 600, 0.1, None, 0)
        ops.attention_decode_ring_fp16_noalloc(dev(q), dev(kc), dev(vc), got, H, KV, hd, 0, 0, 600, 600, 0.1, 0)
        np.testing.assert_allclose(host(got), host(want), **TOL)
    # and where the built-in array, not the sequence length, limits the number of KV splits:
    # H 32 / head_dim 128 allows 262144 / (32 * 130) = 63 splits, a 4096-token context asks for more
    H, KV, hd, cur = 32, 8, 128, 4096
    q, kc, vc = _case(99, H, KV, hd, cur)
    want, got = empty((H, hd)), empty((H, hd))
    ops.attention_decode_ring_fp16(dev(q), dev(kc), dev(vc), want, H, KV, hd, 0, 0, cur, cur, hd ** -0.5, None, 0)
    ops.attention_decode_ring_fp16_noalloc(dev(q), dev(kc), dev(vc), got, H, KV, hd, 0, 0, cur, cur, hd ** -0.5, 0)
    np.testing.assert_allclose(host(got), host(want), **TOL)
    t = empty(1 << 12)
    with pytest.raises(B200Error, match="exceeds the built-in scratch"):
        # H * (hd + 2) = 2048 * 258 floats is beyond the 262144-float array: refused before any launch
        ops.attention_decode_ring_fp16_noalloc(t, t, t, t, 2048, 2048, 256, 0, 0, 1, 1, 0.1, 0)
    with pytest.raises(B200Error, match="exceeds cache"):
        ops.attention_decode_ring_fp16_noalloc(t, t, t, t, 12, 4, 64, 0, 0, 30, 20, 0.1, 0)


def test_noalloc_matches_the_oracle(oracle):
    """Against the CPU restatement of cpu::attention_decode_ring_fp16 (core/attn_cpu.cpp:158-254):
    ring with a pinned prefix and a wrapped start, a window, and the 4096-token / 32-head case in
    which the scratch capacity caps the splits."""
    from gpu_util import dev, empty, host, ops
    for seed, (H, KV, hd), cache_max, rs, pin, cur, win in (
            (5, (12, 4, 128), 512, 37, 8, 300, 0),
            (6, (12, 4, 64), 256, 0, 0, 256, 100),
            (7, (32, 8, 128), 4096, 0, 0, 4096, 0)):
        q, kc, vc = _case(seed, H, KV, hd, cache_max)
        scale = float(hd) ** -0.5
        want = oracle.attention_decode_ring(q, kc, vc, 1, H, KV, hd, rs, pin, cur, cache_max, scale, win)
        got = empty((H, hd))
        ops.attention_decode_ring_fp16_noalloc(dev(q), dev(kc), dev(vc), got, H, KV, hd, rs, pin, cur, cache_max, scale, win)
        np.testing.assert_allclose(host(got), want, **TOL)
