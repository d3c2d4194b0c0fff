"""GPU parity: elementwise ops, embedding, RMSNorm, RoPE, SwiGLU, sampling tail."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_elementwise(oracle):
    from gpu_util import dev, empty, host, ops
    r = np.random.default_rng(0)
    a, b = r.standard_normal(10007).astype(np.float32), r.standard_normal(10007).astype(np.float32)
    out = empty(10007)
    ops.add(dev(a), dev(b), out, 10007)
    assert np.array_equal(host(out), a + b)
    da = dev(a)
    ops.add_inplace(da, dev(b), 10007)
    assert np.array_equal(host(da), a + b)
    ops.scale_inplace(da, 0.22, 10007)
    assert np.array_equal(host(da), (a + b) * np.float32(0.22))
    y = r.standard_normal((7, 33)).astype(np.float32)
    bias = r.standard_normal(33).astype(np.float32)
    dy = dev(y)
    ops.add_bias(dev(bias), dy, 7, 33)
    assert np.array_equal(host(dy), y + bias)
    ops.zero(dy, 7 * 33)
    assert not host(dy).any()
    ops.copy(dy, dev(y), 7 * 33)
    assert np.array_equal(host(dy), y)
    g, u = r.standard_normal(4097).astype(np.float32) * 3, r.standard_normal(4097).astype(np.float32)
    s = empty(4097)
    ops.swiglu_forward(dev(g), dev(u), s, 4097)
    np.testing.assert_allclose(host(s), oracle.swiglu(g, u), rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("half", [False, True])
def test_embedding(oracle, half):
    from gpu_util import dev, empty, host, ops
    r = np.random.default_rng(1)
    vocab, dim = 1000, 96
    tab = r.standard_normal((vocab, dim)).astype(np.float32)
    ids = np.array([0, 999, 5, -1, 1000, 5], np.int32)       # out-of-range ids give zero rows
    out = empty((ids.size, dim))
    if half:
        tabh = oracle.f32_to_f16(tab)
        ops.embedding_forward_half(dev(ids), dev(tabh), out, ids.size, dim, vocab)
        assert np.array_equal(host(out), oracle.embedding(ids, tabh, True, dim, vocab))
    else:
        ops.embedding_forward(dev(ids), dev(tab), out, ids.size, dim, vocab)
        assert np.array_equal(host(out), oracle.embedding(ids, tab, False, dim, vocab))


@pytest.mark.parametrize("rows,dim", [(1, 1536), (5, 768), (64, 128), (3, 100)])
def test_rmsnorm(oracle, rows, dim):
    from gpu_util import dev, empty, host, ops
    r = np.random.default_rng(rows + dim)
    x = (r.standard_normal((rows, dim)) * 3).astype(np.float32)
    w = r.standard_normal(dim).astype(np.float32)
    want, want_rr = oracle.rmsnorm(x, w, 1e-5, True)
    out, rr = empty((rows, dim)), empty(rows)
    ops.rmsnorm_forward(dev(x), dev(w), out, rr, rows, dim, 1e-5)
    np.testing.assert_allclose(host(rr), want_rr, rtol=1e-6)
    np.testing.assert_allclose(host(out), want, rtol=1e-6, atol=1e-7)
    dx = dev(x)                                            # in place (qk-norm, model/model.cpp:2500)
    ops.rmsnorm_forward(dx, dev(w), dx, None, rows, dim, 1e-5)
    np.testing.assert_allclose(host(dx), want, rtol=1e-6, atol=1e-7)
    z = np.zeros((2, dim), np.float32)
    z[1, 0] = np.inf                                       # non-finite inverse becomes 0
    out = empty((2, dim))
    ops.rmsnorm_forward(dev(z), dev(w), out, None, 2, dim, 0.0)
    got = host(out)
    assert not got[0].any() and np.isnan(got[1, 0]) and not got[1, 1:].any()


@pytest.mark.parametrize("rope_type", [0, 1])
def test_rope_cached(oracle, rope_type):
    from gpu_util import dev, host, ops
    r = np.random.default_rng(3)
    ntok, H, KV, hd = 6, 12, 4, 64
    q = r.standard_normal((ntok, H, hd)).astype(np.float32)
    k = r.standard_normal((ntok, KV, hd)).astype(np.float32)
    pos = np.array([0, 1, 2, 127, 1000, 4095], np.int32)
    inv = (1.0 / 10000.0 ** (np.arange(hd // 2) / (hd / 2))).astype(np.float32)
    wq, wk = oracle.rope_cached(q, k, pos, inv, H, KV, hd, rope_type)
    dq, dk = dev(q), dev(k)
    ops.rope_forward_cached(dq, dk, dev(pos), dev(inv), ntok, H, KV, hd, rope_type)
    np.testing.assert_allclose(host(dq), wq, rtol=1e-5, atol=2e-6)
    np.testing.assert_allclose(host(dk), wk, rtol=1e-5, atol=2e-6)


def test_argmax(oracle):
    from gpu_util import dev, ops
    r = np.random.default_rng(4)
    V = 100352
    logits = r.standard_normal(V).astype(np.float32)
    import ctypes
    tok = ctypes.c_int32(-1)
    ops.argmax_token(dev(logits), V, ctypes.addressof(tok))
    assert tok.value == oracle.argmax(logits)
    logits[777] = logits[90000] = logits.max() + 1          # tie -> lowest id
    logits[3], logits[5] = np.nan, np.inf                   # non-finite skipped
    ops.argmax_token(dev(logits), V, ctypes.addressof(tok))
    assert tok.value == oracle.argmax(logits) == 777
    allbad = np.full(1000, np.nan, np.float32)
    allbad[17] = np.inf
    ops.argmax_token(dev(allbad), 1000, ctypes.addressof(tok))
    assert tok.value == oracle.argmax(allbad)
    d = torch.empty(1, dtype=torch.int32, device="cuda")
    ops.argmax_token_device(dev(logits), V, d)
    assert int(d.item()) == 777


def test_topk_and_penalties(oracle):
    from gpu_util import dev, empty, host, ops
    r = np.random.default_rng(5)
    V = 32768
    logits = np.round(r.standard_normal(V) * 4).astype(np.float32) / 4      # many ties
    for K in (1, 8, 40, 128):
        vals, ids = empty(K), empty(K, torch.int32)
        ops.topk_select(dev(logits), V, K, vals, ids)
        wv, wi = oracle.topk(logits, K)
        assert np.array_equal(host(ids), wi) and np.array_equal(host(vals), wv)
    hist = r.integers(-3, V + 3, 700).astype(np.int32)
    hist[:50] = hist[50:100]
    dl = dev(logits)
    ops.apply_rep_penalties(dl, V, dev(hist), hist.size, 1.12, 0.05, 0.3)
    # and with the history in host memory, as the reference's generator passes it
    dl_host_hist = dev(logits)
    ops.apply_rep_penalties(dl_host_hist, V, hist.ctypes.data, hist.size, 1.12, 0.05, 0.3)
    assert np.array_equal(host(dl_host_hist).view(np.uint32), host(dl).view(np.uint32))
    np.testing.assert_allclose(host(dl), oracle.rep_penalties(logits, hist, 1.12, 0.05, 0.3), rtol=1e-6, atol=1e-6)


def test_bounded_wait_runs_out_and_the_library_recovers(oracle):
    """The wait every TMA-fed kernel uses, on a barrier nobody arrives on: it gives up after its
    limit, the kernel returns, b200_stream_status reports the raised word once (B200_ECUDA), and
    the next call runs clean."""
    import torch
    from gpu_util import dev, empty, host, pkg
    lib = pkg.lib()
    assert lib.raw("b200_stream_status") == 0
    outcome = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib.b200_test_bounded_wait(500, outcome)
    assert lib.raw("b200_stream_status") != 0          # the word was raised
    assert "bounded" in lib.last_error().lower() or "wait" in lib.last_error().lower()
    assert int(host(outcome)[0]) == 2                  # the wait returned false, the kernel completed
    assert lib.raw("b200_stream_status") == 0          # read once, cleared
    x = np.random.default_rng(0).standard_normal(1000).astype(np.float32)
    out = empty(1000)
    lib.b200_scale_inplace(dev(x), 2.0, 1000)          # the context is intact
    w = oracle.quantize(np.random.default_rng(1).standard_normal(64 * 256).astype(np.float32) * 0.02, 3)
    y = empty((1, 64))
    xs = np.random.default_rng(2).standard_normal((1, 256)).astype(np.float32)
    lib.b200_linear_forward_q4(dev(xs), dev(w), y, 1, 256, 64, 3)   # a TMA-fed kernel with the same wait
    np.testing.assert_allclose(host(y), oracle.linear(xs, w, 3, 1, 256, 64), rtol=2e-4, atol=2e-5)
    assert lib.raw("b200_stream_status") == 0


def test_phase_timers():
    """cuda_ops.h:315-319: intervals on the stream, reported per phase once complete."""
    import ctypes as C
    import torch
    from gpu_util import pkg
    lib = pkg.lib()
    lib.b200_phase_reset()
    x = torch.zeros(1 << 24, device="cuda")
    lib.b200_phase_start(1)
    for _ in range(20):
        lib.b200_scale_inplace(x, 1.0, x.numel())
    lib.b200_phase_start(0)                    # closes phase 1, opens phase 0
    lib.b200_scale_inplace(x, 1.0, x.numel())
    lib.b200_phase_stop(0)
    lib.b200_phase_start(4)                    # left open: not reported yet
    torch.cuda.synchronize()
    ms = (C.c_double * 5)()
    lib.b200_phase_report(ms, 5)
    assert ms[1] > ms[0] > 0.0 and ms[2] == ms[3] == ms[4] == 0.0
    lib.b200_phase_stop(4)
    torch.cuda.synchronize()
    again = (C.c_double * 5)()
    lib.b200_phase_report(again, 5)
    assert again[0] == again[1] == 0.0 and again[4] > 0.0      # reported intervals are not counted twice
    lib.b200_phase_shutdown()
