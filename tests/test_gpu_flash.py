"""GPU parity: the tensor-core prefill attention (sequences of 128 tokens and more, no
probability output) against the CPU oracle.  q, k, v and the probabilities are rounded
to fp16 inside the kernel, so the bound is relative to the output scale."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run(q, k, v, B, T, H, KV, hd, scale, window, seg):
    from gpu_util import dev, empty, host, ops
    out = empty((B, T, H, hd))
    ops.attention_forward_ex(dev(q), dev(k), dev(v), out, None, B, T, H, KV, hd, scale, window, dev(seg))
    return host(out)


@pytest.mark.parametrize("T,H,KV,hd,window,use_seg", [(128, 4, 2, 64, 0, False), (300, 4, 2, 128, 0, False),
                                                     (257, 6, 2, 64, 37, False), (200, 4, 4, 128, 0, True),
                                                     (1000, 12, 4, 128, 0, False)])
def test_flash_matches_oracle(oracle, T, H, KV, hd, window, use_seg):
    from gpu_util import fp16_close
    B = 2 if T < 1000 else 1
    r = np.random.default_rng(T + hd)
    q = r.standard_normal((B, T, H, hd)).astype(np.float32)
    k = r.standard_normal((B, T, KV, hd)).astype(np.float32)
    v = r.standard_normal((B, T, KV, hd)).astype(np.float32)
    seg = None
    if use_seg:
        seg = np.sort(r.integers(0, 4, (B, T)), axis=1).astype(np.int32)
        seg[1, :50] = -1                       # negative id: that query sees every key
    scale = 1.0 / np.sqrt(hd)
    got = _run(q, k, v, B, T, H, KV, hd, scale, window, seg)
    want = oracle.attention_forward(q, k, v, B, T, H, KV, hd, scale, window, seg)
    assert np.isfinite(got).all()
    fp16_close(got, want, frac=4e-3)


def test_flash_equals_simt_kernel_on_the_same_inputs(oracle):
    """The probability-returning path (exact fp32 kernel) and the flash path agree."""
    from gpu_util import dev, empty, fp16_close, host, ops
    B, T, H, KV, hd = 1, 256, 4, 2, 64
    r = np.random.default_rng(5)
    q = r.standard_normal((B, T, H, hd)).astype(np.float32)
    k = r.standard_normal((B, T, KV, hd)).astype(np.float32)
    v = r.standard_normal((B, T, KV, hd)).astype(np.float32)
    out_a, probs = empty((B, T, H, hd)), empty((B, H, T, T))
    ops.attention_forward_ex(dev(q), dev(k), dev(v), out_a, probs, B, T, H, KV, hd, 0.125, 0, None)
    fp16_close(_run(q, k, v, B, T, H, KV, hd, 0.125, 0, None), host(out_a), frac=4e-3)
    np.testing.assert_allclose(host(probs).sum(-1), 1.0, rtol=1e-5)
