"""Pins the scalar oracle to the reference engine's own CPU objects.

Runs only where oracle/_ref/libgai_ref.so exists (it is built from the mounted
reference sources).  Integer / byte results must be identical; floating-point
results may differ only by summation order (the reference uses an AVX2 tree in
dot_f32 on hosts that have it), hence the small tolerances.
"""
import numpy as np
import pytest

from cases import mamba_case, moe_case


def rng(seed):
    return np.random.default_rng(seed)


@pytest.mark.parametrize("kind", [0, 1, 2])
def test_quantize_and_dequantize_bit_exact(oracle, ref, kind):
    x = (rng(kind).standard_normal(32 * 257) * 0.02).astype(np.float32)
    x[5] = 0.0
    x[64:96] = 0.0                      # an all-zero block (scale 0)
    po, pr = oracle.quantize(x, kind), ref.quantize(x, kind)
    assert np.array_equal(po, pr)
    assert np.array_equal(oracle.dequantize(po, x.size, kind), ref.dequantize(pr, x.size, kind))
    assert np.array_equal(oracle.dequantize_f32(po, x.size, kind).view(np.uint32),
                          ref.dequantize_f32(pr, x.size, kind).view(np.uint32))


@pytest.mark.parametrize("kind", [0, 1, 2])
def test_quantize_non_finite_block(oracle, ref, kind):
    x = rng(7).standard_normal(96).astype(np.float32)
    x[40] = np.inf
    assert np.array_equal(oracle.quantize(x, kind), ref.quantize(x, kind))


def test_fp16_conversion_all_halves(oracle, ref):
    h = np.arange(65536, dtype=np.uint16)
    f = oracle.f16_to_f32(h)
    finite = np.isfinite(f)
    assert np.array_equal(f[finite], h.view(np.float16).astype(np.float32)[finite])
    back = oracle.f32_to_f16(f[finite])
    assert np.array_equal(back, h[finite])
    x = (rng(3).standard_normal(100000) * np.exp(rng(4).uniform(-20, 12, 100000))).astype(np.float32)
    assert np.array_equal(oracle.f32_to_f16(x), x.astype(np.float16).view(np.uint16))


@pytest.mark.parametrize("kind", [0, 1, 2])
def test_linear_q4_bit_exact(oracle, ref, kind):
    M, K, N = 3, 96, 17
    r = rng(10 + kind)
    w = oracle.quantize((r.standard_normal(N * K) * 0.02).astype(np.float32), kind)
    x = r.standard_normal((M, K)).astype(np.float32)
    a, b = oracle.linear(x, w, kind, M, K, N), ref.linear(x, w, kind, M, K, N)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_linear_f16_f32(oracle, ref):
    M, K, N = 2, 200, 33
    r = rng(20)
    x = r.standard_normal((M, K)).astype(np.float32)
    wf = (r.standard_normal((N, K)) * 0.05).astype(np.float32)
    wh = wf.astype(np.float16).view(np.uint16)
    a, b = oracle.linear(x, wh, -1, M, K, N), ref.linear(x, wh, -1, M, K, N)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    np.testing.assert_allclose(oracle.linear(x, wf, -2, M, K, N), ref.linear(x, wf, -2, M, K, N),
                               rtol=1e-5, atol=1e-6)


def test_small_ops(oracle, ref):
    r = rng(30)
    x = r.standard_normal((5, 96)).astype(np.float32)
    w = r.standard_normal(96).astype(np.float32)
    for a, b in zip(oracle.rmsnorm(x, w, 1e-5, True), ref.rmsnorm(x, w, 1e-5, True)):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    g, u = r.standard_normal(300).astype(np.float32), r.standard_normal(300).astype(np.float32)
    assert np.array_equal(oracle.swiglu(g, u).view(np.uint32), ref.swiglu(g, u).view(np.uint32))
    tab = r.standard_normal((50, 16)).astype(np.float32)
    ids = np.array([0, 49, -1, 50, 7], np.int32)
    assert np.array_equal(oracle.embedding(ids, tab, False, 16, 50), ref.embedding(ids, tab, False, 16, 50))
    tabh = tab.astype(np.float16).view(np.uint16)
    assert np.array_equal(oracle.embedding(ids, tabh, True, 16, 50), ref.embedding(ids, tabh, True, 16, 50))
    for rope_type in (0, 1):
        q = r.standard_normal((4, 6, 32)).astype(np.float32)
        k = r.standard_normal((4, 2, 32)).astype(np.float32)
        pos = np.array([0, 1, 77, 4095], np.int32)
        inv = (1.0 / 10000.0 ** (np.arange(16) / 16.0)).astype(np.float32)
        qa, ka = oracle.rope_cached(q, k, pos, inv, 6, 2, 32, rope_type)
        qb, kb = ref.rope_cached(q, k, pos, inv, 6, 2, 32, rope_type)
        assert np.array_equal(qa.view(np.uint32), qb.view(np.uint32))
        assert np.array_equal(ka.view(np.uint32), kb.view(np.uint32))


def test_sampling_tail(oracle, ref):
    r = rng(40)
    logits = r.standard_normal(1000).astype(np.float32)
    logits[10] = logits[500] = logits.max() + 1.0          # tie -> lowest id
    logits[3] = np.nan
    logits[4] = np.inf
    assert oracle.argmax(logits) == ref.argmax(logits) == 10
    clean = np.where(np.isfinite(logits), logits, 0).astype(np.float32)
    va, ia = oracle.topk(clean, 8)
    vb, ib = ref.topk(clean, 8)
    assert np.array_equal(ia, ib) and np.array_equal(va, vb)
    hist = np.array([10, 10, 999, -5, 2000, 7], np.int32)
    a = oracle.rep_penalties(clean, hist, 1.12, 0.1, 0.2)
    b = ref.rep_penalties(clean, hist, 1.12, 0.1, 0.2)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


@pytest.mark.parametrize("wkind", [-2, -1, 2, 0])
def test_moe_forward(oracle, ref, wkind):
    c = moe_case(oracle, seed=50, N=9, d=64, E=32, ne=8, K=2, SH=64, wkind=wkind, bias_sigma=0.02)
    args = (c["x"], c["router_w"], c["router_bias"], c["gates"], c["ups"], c["downs"],
            c["sh_g"], c["sh_u"], c["sh_d"], 64, 32, 8, 2, 64, wkind)
    oa, pa, ia, wa = oracle.moe_forward(*args)
    ob, pb, ib, wb = ref.moe_forward(*args)
    assert np.array_equal(ia, ib)                                   # routing bit-exact
    assert np.array_equal(pa.view(np.uint32), pb.view(np.uint32))
    assert np.array_equal(wa.view(np.uint32), wb.view(np.uint32))
    np.testing.assert_allclose(oa, ob, rtol=2e-5, atol=2e-6)


def test_moe_forward_no_shared_K8(oracle, ref):
    c = moe_case(oracle, seed=51, N=5, d=32, E=32, ne=64, K=8, SH=0, wkind=-2, bias_sigma=0.0)
    args = (c["x"], c["router_w"], None, c["gates"], c["ups"], c["downs"], None, None, None,
            32, 32, 64, 8, 0, -2)
    oa, pa, ia, wa = oracle.moe_forward(*args)
    ob, pb, ib, wb = ref.moe_forward(*args)
    assert np.array_equal(ia, ib)
    assert np.array_equal(wa.view(np.uint32), wb.view(np.uint32))
    np.testing.assert_allclose(oa, ob, rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("wkind", [-2, -1, 2, 1])
def test_mamba2_forward(oracle, ref, wkind):
    c = mamba_case(oracle, seed=60, B=2, T=7, d=64, n_heads=4, d_head=32, d_state=16, k=4, wkind=wkind)
    oa, sa = oracle.mamba2_forward(*c["args"], wkind)
    ob, sb = ref.mamba2_forward(*c["args"], wkind)
    np.testing.assert_allclose(oa, ob, rtol=2e-5, atol=2e-6)
    np.testing.assert_allclose(sa, sb, rtol=2e-5, atol=2e-7)


def test_mamba2_step_equals_forward_T1_chain(oracle):
    """The decode step (carried conv window) walked T times equals one forward over T
    with a zero window: ties the restated step (which the reference only has as a
    private member on its host path) to the pinned forward."""
    c = mamba_case(oracle, seed=61, B=1, T=6, d=64, n_heads=4, d_head=32, d_state=16, k=4, wkind=2)
    (x, w_in, conv_w, conv_b, dt_bias, a_log, D, norm_w, w_out, state,
     B, T, d, d_inner, conv_dim, n_heads, d_head, d_state, k, eps) = c["args"]
    full, s_full = oracle.mamba2_forward(*c["args"], 2)
    conv_state = np.zeros((conv_dim, k - 1), np.float32)
    s = state.copy()
    for t in range(T):
        y, conv_state, s = oracle.mamba2_step(x[0, t], w_in, conv_w, conv_b, dt_bias, a_log, D,
                                              norm_w, w_out, conv_state, s, d, d_inner, conv_dim,
                                              n_heads, d_head, d_state, k, eps, 2)
        assert np.array_equal(y.view(np.uint32), full[0, t].view(np.uint32))
    assert np.array_equal(s.view(np.uint32), s_full.view(np.uint32))


def test_attention(oracle, ref):
    r = rng(70)
    B, T, H, KV, hd = 2, 9, 4, 2, 16
    q = r.standard_normal((B, T, H, hd)).astype(np.float32)
    k = r.standard_normal((B, T, KV, hd)).astype(np.float32)
    v = r.standard_normal((B, T, KV, hd)).astype(np.float32)
    seg = np.array([[0, 0, 0, 1, 1, 1, 1, 2, 2], [0] * 9], np.int32)
    for window, s in ((0, None), (3, None), (0, seg)):
        oa, pa = oracle.attention_forward(q, k, v, B, T, H, KV, hd, 0.25, window, s, True)
        ob, pb = ref.attention_forward(q, k, v, B, T, H, KV, hd, 0.25, window, s, True)
        np.testing.assert_allclose(oa, ob, rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(pa, pb, rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("half", [0, 1])
def test_attention_decode_ring(oracle, ref, half):
    r = rng(80 + half)
    H, KV, hd, cache_max = 6, 2, 32, 24
    q = r.standard_normal((H, hd)).astype(np.float32)
    kc = r.standard_normal((cache_max, KV * hd)).astype(np.float32)
    vc = r.standard_normal((cache_max, KV * hd)).astype(np.float32)
    if half:
        kc, vc = kc.astype(np.float16).view(np.uint16), vc.astype(np.float16).view(np.uint16)
    for ring_start, pinned, cur_len, window in ((0, 0, 1, 0), (0, 0, 24, 0), (5, 4, 24, 0),
                                                (0, 0, 17, 6), (3, 0, 20, 0)):
        a = oracle.attention_decode_ring(q, kc, vc, half, H, KV, hd, ring_start, pinned, cur_len,
                                         cache_max, 0.2, window)
        b = ref.attention_decode_ring(q, kc, vc, half, H, KV, hd, ring_start, pinned, cur_len,
                                      cache_max, 0.2, window)
        np.testing.assert_allclose(a, b, rtol=1e-5, atol=1e-6)
    for bad in ((0, 0, 25, 24), (0, 30, 10, 24)):   # cur_len > cache_max, pinned > cur_len
        with pytest.raises(ValueError):
            oracle.attention_decode_ring(q, kc, vc, half, H, KV, hd, bad[0], bad[1], bad[2], bad[3], 0.2)
        with pytest.raises(ValueError):
            ref.attention_decode_ring(q, kc, vc, half, H, KV, hd, bad[0], bad[1], bad[2], bad[3], 0.2)
