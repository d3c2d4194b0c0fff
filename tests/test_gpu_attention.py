"""GPU parity: ring / paged decode attention and causal prefill attention."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = dict(rtol=2e-4, atol=2e-5)


@pytest.mark.parametrize("half", [0, 1])
@pytest.mark.parametrize("H,KV,hd", [(12, 4, 64), (12, 4, 128), (32, 8, 128), (4, 4, 32), (16, 1, 64)])
def test_decode_ring(oracle, half, H, KV, hd):
    from gpu_util import dev, empty, host, ops
    r = np.random.default_rng(H + hd + half)
    cache_max = 700
    q = r.standard_normal((H, hd)).astype(np.float32)
    kc = r.standard_normal((cache_max, KV * hd)).astype(np.float32)
    vc = r.standard_normal((cache_max, KV * hd)).astype(np.float32)
    if half:
        kc, vc = oracle.f32_to_f16(kc), oracle.f32_to_f16(vc)
    dq, dk, dv = dev(q), dev(kc), dev(vc)
    fn = ops.attention_decode_ring_fp16 if half else ops.attention_decode_ring
    # (ring_start, pinned, cur_len, window)
    for rs, pin, cur, win in ((0, 0, 1, 0), (0, 0, 2, 0), (0, 0, 700, 0), (123, 8, 700, 0), (0, 0, 333, 100),
                              (691, 8, 500, 0), (0, 0, 0, 0), (5, 0, 64, 64)):
        want = oracle.attention_decode_ring(q, kc, vc, half, H, KV, hd, rs, pin, cur, cache_max, hd ** -0.5, win)
        out = empty((H, hd))
        fn(dq, dk, dv, out, H, KV, hd, rs, pin, cur, cache_max, hd ** -0.5, None, win)
        np.testing.assert_allclose(host(out), want, **TOL)


def test_decode_ring_long_context(oracle):
    """H-Tiny attention layer at ctx 4096 (fp16 cache)."""
    from gpu_util import dev, empty, host, ops
    r = np.random.default_rng(1)
    H, KV, hd, n = 12, 4, 128, 4096
    q = r.standard_normal((H, hd)).astype(np.float32)
    kc = oracle.f32_to_f16(r.standard_normal((n, KV * hd)).astype(np.float32))
    vc = oracle.f32_to_f16(r.standard_normal((n, KV * hd)).astype(np.float32))
    want = oracle.attention_decode_ring(q, kc, vc, 1, H, KV, hd, 0, 0, n, n, hd ** -0.5, 0)
    out = empty((H, hd))
    ops.attention_decode_ring_fp16(dev(q), dev(kc), dev(vc), out, H, KV, hd, 0, 0, n, n, hd ** -0.5, None, 0)
    np.testing.assert_allclose(host(out), want, **TOL)


def test_decode_ring_errors(oracle):
    from gpu_util import B200Error, empty, ops
    t = empty(1 << 14)
    for args, msg in (((12, 5, 64, 0, 0, 10, 20), "multiple of KV"), ((12, 4, 64, 0, 0, 30, 20), "exceeds cache"),
                      ((12, 4, 64, 0, 11, 10, 20), "pinned prefix"), ((12, 4, 64, 25, 0, 10, 20), "ring start"),
                      ((12, 4, 64, 0, 10, 15, 10), "exceeds cache")):
        with pytest.raises(B200Error, match=msg):
            ops.attention_decode_ring(t, t, t, t, *args, 0.1, None, 0)


def test_decode_paged_ragged_batch(oracle):
    """64 sequences with ragged lengths over a shuffled page pool (block 64) == per-sequence
    ring-cache oracle on each sequence's contiguous copy."""
    from gpu_util import dev, empty, host, ops
    r = np.random.default_rng(7)
    batch, H, KV, hd, page = 64, 12, 4, 128, 64
    lens = r.integers(1, 1500, batch).astype(np.int32)
    lens[0], lens[1] = 1, 64
    max_pages = int((lens.max() + page - 1) // page)
    need = [(int(l) + page - 1) // page for l in lens]
    pool = r.permutation(sum(need) + 5)
    table = np.zeros((batch, max_pages), np.int32)
    k_pages = np.zeros((sum(need) + 5, page, KV * hd), np.uint16)
    v_pages = np.zeros_like(k_pages)
    q = r.standard_normal((batch, H, hd)).astype(np.float32)
    want = np.zeros((batch, H, hd), np.float32)
    pi = 0
    for b in range(batch):
        kc = oracle.f32_to_f16(r.standard_normal((need[b] * page, KV * hd)).astype(np.float32))
        vc = oracle.f32_to_f16(r.standard_normal((need[b] * page, KV * hd)).astype(np.float32))
        for p in range(need[b]):
            table[b, p] = pool[pi]
            k_pages[pool[pi]] = kc[p * page:(p + 1) * page]
            v_pages[pool[pi]] = vc[p * page:(p + 1) * page]
            pi += 1
        want[b] = oracle.attention_decode_ring(q[b], kc, vc, 1, H, KV, hd, 0, 0, int(lens[b]), need[b] * page,
                                               hd ** -0.5, 0)
    out = empty((batch, H, hd))
    ops.attention_decode_paged_fp16(dev(q), dev(k_pages), dev(v_pages), dev(table), dev(lens), out, batch,
                                    max_pages, page, H, KV, hd, hd ** -0.5)
    np.testing.assert_allclose(host(out), want, **TOL)


@pytest.mark.parametrize("B,T,H,KV,hd", [(1, 1, 4, 2, 32), (2, 37, 12, 4, 64), (1, 130, 12, 4, 128)])
def test_prefill(oracle, B, T, H, KV, hd):
    from gpu_util import dev, empty, host, ops
    r = np.random.default_rng(B + T)
    q = r.standard_normal((B, T, H, hd)).astype(np.float32)
    k = r.standard_normal((B, T, KV, hd)).astype(np.float32)
    v = r.standard_normal((B, T, KV, hd)).astype(np.float32)
    seg = np.sort(r.integers(0, 3, (B, T)), axis=1).astype(np.int32)
    for window, s in ((0, None), (5, None), (0, seg)):
        want, wp = oracle.attention_forward(q, k, v, B, T, H, KV, hd, hd ** -0.5, window, s, True)
        out, probs = empty((B, T, H, hd)), empty((B, H, T, T))
        ops.attention_forward_ex(dev(q), dev(k), dev(v), out, probs, B, T, H, KV, hd, hd ** -0.5, window, dev(s))
        np.testing.assert_allclose(host(out), want, **TOL)
        np.testing.assert_allclose(host(probs), wp, rtol=2e-4, atol=1e-6)
        out2 = empty((B, T, H, hd))
        ops.attention_forward_ex(dev(q), dev(k), dev(v), out2, None, B, T, H, KV, hd, hd ** -0.5, window, dev(s))
        if T < 128:
            assert np.array_equal(host(out2), host(out))     # same kernel with and without the probabilities
        else:
            from gpu_util import fp16_close                  # 128 tokens and more: tensor-core kernel
            fp16_close(host(out2), host(out), frac=4e-3)
