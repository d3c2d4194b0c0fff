"""GPU parity: MoE routing (bit-exact), expert permutation (bit-exact), layer output."""
import numpy as np
import pytest
import torch

from cases import moe_case

pytestmark = pytest.mark.gpu


def _run(c, N, d, E, ne, K, SH, wkind, caches=True, scratch=False):
    from gpu_util import dev, empty, host, ops
    out = empty((N, d))
    probs = empty((N, ne)) if caches else None
    idx = empty((N, K), torch.int32) if caches else None
    w = empty((N, K)) if caches else None
    sg = empty((N, K, E)) if scratch else None
    su = empty((N, K, E)) if scratch else None
    sa = empty((N, K, E)) if scratch else None
    args = [dev(c[k]) for k in ("gates", "ups", "downs", "sh_g", "sh_u", "sh_d")]
    if wkind == -2:
        ops.moe_forward_bias(dev(c["x"]), dev(c["router_w"]), dev(c["router_bias"]), *args, out, probs, idx, w,
                             sg, su, sa, N, d, E, ne, K, SH)
    else:
        ops.moe_forward_bias_half(dev(c["x"]), dev(c["router_w"]), dev(c["router_bias"]), *args, out, probs, idx,
                                  w, sg, su, sa, N, d, E, ne, K, SH, wkind)
    res = dict(out=host(out))
    if caches:
        res.update(probs=host(probs), idx=host(idx), w=host(w))
    if scratch:
        res.update(sg=host(sg), su=host(su), sa=host(sa))
    return res


def _ulp_close(a, b, maxulp=4):
    """Router probabilities / mixture weights.  Logits follow the reference's fp32 chain
    bit for bit; exp() is evaluated in double and rounded, which differs from the host
    libm's expf by one ulp for a fraction of a percent of arguments, and the softmax
    sum can carry that ulp into every probability of the row."""
    np.testing.assert_array_max_ulp(a, b, maxulp=maxulp)


def _close(got, want, N, wkind):
    """From 32 tokens on, fp16 / packed experts run as tensor-core GEMMs on fp16 copies
    of the activations (and of the dequantised weights): compared relative to the
    output scale.  Fewer tokens and fp32 experts stay in fp32: summation-order bound."""
    from gpu_util import SUM_ORDER
    if N >= 32 and wkind != -2:
        scale = float(np.abs(want).max())
        assert float(np.abs(got - want).max()) <= 4e-3 * scale, (float(np.abs(got - want).max()), scale)
    else:
        np.testing.assert_allclose(got, want, **SUM_ORDER)


def _oracle(oracle, c, d, E, ne, K, SH, wkind):
    return oracle.moe_forward(c["x"], c["router_w"], c["router_bias"], c["gates"], c["ups"], c["downs"],
                              c["sh_g"], c["sh_u"], c["sh_d"], d, E, ne, K, SH, wkind)


@pytest.mark.parametrize("wkind", [-2, -1, 0, 1, 2, 3])
@pytest.mark.parametrize("N", [1, 5, 64])
def test_layer_small(oracle, wkind, N):
    from gpu_util import SUM_ORDER
    d, E, ne, K, SH = 256, 256, 16, 2, 512
    c = moe_case(oracle, 10 * N + wkind + 3, N, d, E, ne, K, SH, wkind)
    got = _run(c, N, d, E, ne, K, SH, wkind)
    out, probs, idx, w = _oracle(oracle, c, d, E, ne, K, SH, wkind)
    assert np.array_equal(got["idx"], idx)                                # top-k indices bit-exact
    _ulp_close(got["probs"], probs)
    _ulp_close(got["w"], w)
    _close(got["out"], out, N, wkind)


@pytest.mark.parametrize("N", [1, 64, 512])
def test_layer_config3_shape(oracle, N):
    """hidden 1536, 64 experts, top-6, ffn 512, shared 1024, Q4_K, skewed router bias."""
    d, E, ne, K, SH = 1536, 512, 64, 6, 1024
    c = moe_case(oracle, 300 + N, N, d, E, ne, K, SH, 3)
    got = _run(c, N, d, E, ne, K, SH, 3)
    out, probs, idx, w = _oracle(oracle, c, d, E, ne, K, SH, 3)
    assert np.array_equal(got["idx"], idx)
    _ulp_close(got["w"], w)
    _close(got["out"], out, N, 3)


@pytest.mark.parametrize("wkind", [3, 2, 0, -1])
@pytest.mark.parametrize("N", [9, 33, 128])
def test_layer_decode_batch_without_shared_expert_is_fp32_tight(oracle, wkind, N):
    """A decode batch (more than 8 tokens, at most ~12 rows per expert) runs the routed experts
    as weight streams shared by their tokens, on the few-token dot engine: exact dequantised
    weights, fp32 accumulation - the summation-order bound, not the fp16 one.  Without a
    shared expert nothing in the layer touches the tensor-core GEMM.  Ragged loads: the router
    bias sends up to a few dozen tokens to one expert (several units) and none to others."""
    from gpu_util import SUM_ORDER
    d, E, ne, K, SH = 512, 256, 64, 6, 0
    c = moe_case(oracle, 900 + N + wkind, N, d, E, ne, K, 0, wkind, bias_sigma=0.05)
    got = _run(c, N, d, E, ne, K, SH, wkind)
    out, probs, idx, w = _oracle(oracle, c, d, E, ne, K, SH, wkind)
    assert np.array_equal(got["idx"], idx)
    _ulp_close(got["w"], w)
    np.testing.assert_allclose(got["out"], out, **SUM_ORDER)
    again = _run(c, N, d, E, ne, K, SH, wkind)
    assert np.array_equal(got["out"].view(np.uint32), again["out"].view(np.uint32))      # run-to-run bit-stable


def test_layer_config3_4096_tokens(oracle):
    """The prefill-sized case: routing checked on every token, outputs on a sample of
    tokens (a token's output depends on no other token), and run-to-run bit stability."""
    d, E, ne, K, SH = 1536, 512, 64, 6, 1024
    N = 4096
    c = moe_case(oracle, 4096, N, d, E, ne, K, SH, 3)
    got = _run(c, N, d, E, ne, K, SH, 3)
    again = _run(c, N, d, E, ne, K, SH, 3)
    assert np.array_equal(got["out"].view(np.uint32), again["out"].view(np.uint32))
    probs, idx, w = oracle.moe_route(c["x"], c["router_w"], c["router_bias"], ne, K)
    assert np.array_equal(got["idx"], idx)
    _ulp_close(got["w"], w)
    sample = np.array([0, 1, 127, 128, 2047, 4000, 4095])
    sub = dict(c, x=np.ascontiguousarray(c["x"][sample]))
    out, _, sidx, _ = _oracle(oracle, sub, d, E, ne, K, SH, 3)
    assert np.array_equal(sidx, idx[sample])
    _close(got["out"][sample], out, N, 3)


@pytest.mark.parametrize("N", [1, 64])
def test_layer_h_small_shape(oracle, N):
    """The widest configuration of the benchmark list: hidden 4096, 72 experts, top-10, expert
    ffn 768, shared ffn 1536, Q4_K (beyond the reference kernels' 64-expert / top-8 limits).
    Indices bit-exact, outputs within the tolerance of their path."""
    d, E, ne, K, SH = 4096, 768, 72, 10, 1536
    c = moe_case(oracle, 5000 + N, N, d, E, ne, K, SH, 3)
    got = _run(c, N, d, E, ne, K, SH, 3)
    out, probs, idx, w = _oracle(oracle, c, d, E, ne, K, SH, 3)
    assert np.array_equal(got["idx"], idx)
    _ulp_close(got["w"], w)
    _close(got["out"], out, N, 3)


def test_routing_bit_exact_many_tokens(oracle):
    """4096 tokens at the config-3 router shape: every top-k index identical, probabilities
    and weights within a few ulp."""
    from gpu_util import dev, empty, host, ops
    d, ne, K = 1536, 64, 6
    r = np.random.default_rng(42)
    x = r.standard_normal((4096, d)).astype(np.float32)
    rw = (r.standard_normal((ne, d)) / np.sqrt(d)).astype(np.float32)
    bias = (r.standard_normal(ne) * 0.5 / ne).astype(np.float32)
    probs, idx, w = oracle.moe_route(x, rw, bias, ne, K)
    # drive the router alone through a layer whose experts are tiny
    E = 32
    z = np.zeros((ne * E, d), np.float32)
    zd = np.zeros((ne * d, E), np.float32)
    out, dp, di, dw = empty((4096, d)), empty((4096, ne)), empty((4096, K), torch.int32), empty((4096, K))
    ops.moe_forward_bias(dev(x), dev(rw), dev(bias), dev(z), dev(z), dev(zd), None, None, None, out, dp, di, dw,
                         None, None, None, 4096, d, E, ne, K, 0)
    assert np.array_equal(host(di), idx)
    _ulp_close(host(dp), probs)
    _ulp_close(host(dw), w)
    # the logits themselves are bit-identical (same fp32 chain); only exp differs
    exact = (host(dp).view(np.uint32) == probs.view(np.uint32)).mean()
    assert exact > 0.98, f"only {exact:.4f} of the probabilities are bit-identical"
    assert not host(out).any()


@pytest.mark.parametrize("d,ne,K", [(1536, 64, 6), (4096, 72, 10), (256, 10, 2)])
def test_routing_bit_exact_decode_batches(oracle, d, ne, K):
    """Token counts around the decode-batch router (8 x 8 chains per block, the finish folded into
    the last block of a token group; 16 to 256 tokens) and its neighbours: indices identical,
    probabilities and weights within a few ulp, expert counts that are no multiple of 8."""
    from gpu_util import dev, empty, host, ops
    r = np.random.default_rng(d + ne)
    rw = (r.standard_normal((ne, d)) / np.sqrt(d)).astype(np.float32)
    bias = (r.standard_normal(ne) * 0.5 / ne).astype(np.float32)
    for N in (15, 16, 17, 100, 255, 256, 257):
        x = r.standard_normal((N, d)).astype(np.float32)
        probs, idx, w = oracle.moe_route(x, rw, bias, ne, K)
        dp, di, dw = empty((N, ne)), empty((N, K), torch.int32), empty((N, K))
        for _ in range(2):          # twice: the arrival counters must be back at zero
            ops.moe_route(dev(x), dev(rw), dev(bias), dp, di, dw, N, d, ne, K)
            assert np.array_equal(host(di), idx), N
            _ulp_close(host(dp), probs)
            _ulp_close(host(dw), w)


def test_routing_ties_and_degenerate(oracle):
    """Identical router rows give exact ties (lowest index wins); huge negative bias and
    underflowing probabilities exercise the uniform-weight fallback."""
    from gpu_util import dev, empty, host, ops
    d, ne, K, E = 64, 8, 3, 32
    r = np.random.default_rng(9)
    x = r.standard_normal((6, d)).astype(np.float32)
    rw = np.tile(r.standard_normal((1, d)).astype(np.float32), (ne, 1))     # all experts tie
    rw[5] *= 1.5
    bias = np.zeros(ne, np.float32)
    x[4] *= 1e4            # softmax saturates: one prob 1, the rest underflow to 0
    z, zd = np.zeros((ne * E, d), np.float32), np.zeros((ne * d, E), np.float32)
    for b in (bias, None, np.full(ne, -2e30, np.float32)):
        probs, idx, w = oracle.moe_route(x, rw, b, ne, K)
        out, di, dw = empty((6, d)), empty((6, K), torch.int32), empty((6, K))
        ops.moe_forward_bias(dev(x), dev(rw), dev(b), dev(z), dev(z), dev(zd), None, None, None, out, None, di,
                             dw, None, None, None, 6, d, E, ne, K, 0)
        assert np.array_equal(host(di), idx)
        _ulp_close(host(dw), w)


def test_wide_config5_limits(oracle):
    """72 experts, top-10: beyond the reference's ne <= 64 / K <= 8 arrays."""
    from gpu_util import SUM_ORDER
    d, E, ne, K, SH = 256, 256, 72, 10, 256
    c = moe_case(oracle, 55, 7, d, E, ne, K, SH, 3)
    got = _run(c, 7, d, E, ne, K, SH, 3)
    out, probs, idx, w = _oracle(oracle, c, d, E, ne, K, SH, 3)
    assert np.array_equal(got["idx"], idx)
    np.testing.assert_allclose(got["out"], out, **SUM_ORDER)


def test_no_shared_k1_and_scratch_outputs(oracle):
    from gpu_util import SUM_ORDER, dev, host
    d, E, ne, K = 128, 64, 4, 1
    c = moe_case(oracle, 66, 9, d, E, ne, K, 0, -2)
    got = _run(c, 9, d, E, ne, K, 0, -2, caches=False, scratch=True)
    out, probs, idx, w = _oracle(oracle, c, d, E, ne, K, 0, -2)
    np.testing.assert_allclose(got["out"], out, **SUM_ORDER)
    # s_gate / s_up / s_act hold the selected experts' pre-activations and activations
    x = c["x"]
    for t in range(9):
        e = idx[t, 0]
        g = c["gates"].reshape(ne, E, d)[e] @ x[t]
        u = c["ups"].reshape(ne, E, d)[e] @ x[t]
        np.testing.assert_allclose(got["sg"][t, 0], g, rtol=1e-4, atol=1e-5)
        np.testing.assert_allclose(got["su"][t, 0], u, rtol=1e-4, atol=1e-5)
        np.testing.assert_allclose(got["sa"][t, 0], oracle.swiglu(g, u), rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("NK,ne", [(1, 4), (6, 64), (384, 64), (1000, 72), (1024, 256), (1025, 64), (4096 * 6, 64), (100003, 72),
                                   (64 * 4096 * 6, 64)])
def test_permutation_bit_exact(oracle, NK, ne):
    """Stable counting sort by expert; the largest case is batch-64 x 4096-token prefill."""
    from gpu_util import dev, empty, host, ops
    r = np.random.default_rng(NK % 1000 + ne)
    p = r.dirichlet(np.full(ne, 0.3))                 # skewed loads, some experts (nearly) empty
    idx = r.choice(ne, size=NK, p=p).astype(np.int32)
    grouped, offsets = empty(NK, torch.int32), empty(ne + 1, torch.int32)
    ops.moe_permutation(dev(idx), NK, ne, grouped, offsets)
    g, o = host(grouped), host(offsets)
    if NK <= 200000:
        wg, wo = oracle.moe_permutation(idx, ne)
        assert np.array_equal(o, wo) and np.array_equal(g, wg)
    # size-independent properties
    assert o[0] == 0 and o[-1] == NK and np.array_equal(np.diff(o), np.bincount(idx, minlength=ne))
    assert np.array_equal(np.sort(g), np.arange(NK))
    ge = idx[g]
    assert (np.diff(ge) >= 0).all()
    same = np.diff(ge) == 0
    assert (np.diff(g)[same] > 0).all()               # ascending slot id inside an expert


def test_argument_errors(oracle):
    from gpu_util import B200Error, empty, ops
    t = empty(1 << 16)
    with pytest.raises(B200Error, match="K must be in"):
        ops.moe_forward_bias(t, t, None, t, t, t, None, None, None, t, None, None, None, None, None, None,
                             1, 64, 32, 8, 0, 0)
    with pytest.raises(B200Error, match="ne out of range"):
        ops.moe_forward_bias(t, t, None, t, t, t, None, None, None, t, None, None, None, None, None, None,
                             1, 64, 32, 300, 2, 0)
    with pytest.raises(B200Error, match="unknown qkind"):
        ops.moe_forward_bias_half(t, t, None, t, t, t, None, None, None, t, None, None, None, None, None, None,
                                  1, 64, 32, 8, 2, 0, 5)
    ops.moe_forward_bias(t, t, None, t, t, t, None, None, None, t, None, None, None, None, None, None,
                         0, 64, 32, 8, 2, 0)          # N == 0 returns silently
