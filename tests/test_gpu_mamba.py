"""GPU parity: Mamba-2 decode step (single and batched) and sequence forward."""
import numpy as np
import pytest
import torch

from cases import mamba_case

pytestmark = pytest.mark.gpu

STATE_TOL = dict(rtol=2e-4, atol=2e-6)


def _dev_params(a):
    from gpu_util import dev
    return [dev(v) for v in a]


@pytest.mark.parametrize("wkind", [-2, -1, 0, 1, 2, 3])
def test_step_chain(oracle, wkind):
    """Eight consecutive decode steps: outputs, conv window and ssm state track the oracle."""
    from gpu_util import SUM_ORDER, dev, empty, host, ops
    c = mamba_case(oracle, 100 + wkind, B=1, T=8, d=256, n_heads=4, d_head=64, d_state=128, k=4, wkind=wkind)
    (x, w_in, conv_w, conv_b, dt_bias, a_log, D, norm_w, w_out, state,
     _, T, d, d_inner, conv_dim, n_heads, d_head, d_state, k, eps) = c["args"]
    cs = np.zeros((conv_dim, k - 1), np.float32)
    ss = state[0].reshape(-1, d_state).copy()
    dcs, dss = dev(cs), dev(ss)
    pw = _dev_params((w_in, conv_w, conv_b, dt_bias, a_log, D, norm_w, w_out))
    for t in range(T):
        want, cs, ss = oracle.mamba2_step(x[0, t], w_in, conv_w, conv_b, dt_bias, a_log, D, norm_w, w_out,
                                          cs, ss, d, d_inner, conv_dim, n_heads, d_head, d_state, k, eps, wkind)
        out = empty(d)
        if wkind == -2:
            ops.mamba2_step(dev(x[0, t]), pw[0], pw[1], pw[2], pw[3], pw[4], pw[5], pw[6], pw[7], dcs, dss, out,
                            d, d_inner, conv_dim, n_heads, d_head, d_state, k, eps)
        else:
            ops.mamba2_step_half(dev(x[0, t]), pw[0], pw[1], pw[2], pw[3], pw[4], pw[5], pw[6], pw[7], dcs, dss,
                                 out, d, d_inner, conv_dim, n_heads, d_head, d_state, k, eps, wkind)
        np.testing.assert_allclose(host(out), want, **SUM_ORDER)
        np.testing.assert_allclose(host(dcs), cs, **SUM_ORDER)
        np.testing.assert_allclose(host(dss), ss, **STATE_TOL)


@pytest.mark.parametrize("shape", [dict(d=768, n_heads=24, d_head=64, d_state=64),      # config 1
                                   dict(d=1536, n_heads=48, d_head=64, d_state=128)])    # H-Tiny
def test_step_model_shapes(oracle, shape):
    from gpu_util import SUM_ORDER, dev, empty, host, ops
    wkind = 2 if shape["d"] == 768 else 3
    c = mamba_case(oracle, 7, B=1, T=1, k=4, wkind=wkind, w_std=0.02, **shape)
    (x, w_in, conv_w, conv_b, dt_bias, a_log, D, norm_w, w_out, state,
     _, _, d, d_inner, conv_dim, n_heads, d_head, d_state, k, eps) = c["args"]
    r = np.random.default_rng(8)
    cs = r.standard_normal((conv_dim, k - 1)).astype(np.float32)
    ss = state[0].reshape(-1, d_state)
    want, wcs, wss = oracle.mamba2_step(x[0, 0], w_in, conv_w, conv_b, dt_bias, a_log, D, norm_w, w_out, cs, ss,
                                        d, d_inner, conv_dim, n_heads, d_head, d_state, k, eps, wkind)
    dcs, dss, out = dev(cs), dev(ss), empty(d)
    ops.mamba2_step_half(dev(x[0, 0]), *_dev_params((w_in, conv_w, conv_b, dt_bias, a_log, D, norm_w, w_out)),
                         dcs, dss, out, d, d_inner, conv_dim, n_heads, d_head, d_state, k, eps, wkind)
    np.testing.assert_allclose(host(out), want, **SUM_ORDER)
    np.testing.assert_allclose(host(dss), wss, **STATE_TOL)
    np.testing.assert_allclose(host(dcs), wcs, **SUM_ORDER)


@pytest.mark.parametrize("batch", [2, 8, 11, 64])
def test_step_batched(oracle, batch):
    """batch independent sequences == batch single-sequence oracle steps."""
    from gpu_util import SUM_ORDER, close, dev, empty, host, ops
    c = mamba_case(oracle, 200 + batch, B=batch, T=1, d=256, n_heads=4, d_head=64, d_state=128, k=4, wkind=3)
    (x, w_in, conv_w, conv_b, dt_bias, a_log, D, norm_w, w_out, state,
     _, _, d, d_inner, conv_dim, n_heads, d_head, d_state, k, eps) = c["args"]
    r = np.random.default_rng(batch)
    cs = r.standard_normal((batch, conv_dim, k - 1)).astype(np.float32)
    ss = state.reshape(batch, -1, d_state)
    dcs, dss, out = dev(cs), dev(ss), empty((batch, d))
    ops.mamba2_step_batched(dev(x[:, 0]), *_dev_params((w_in, conv_w, conv_b, dt_bias, a_log, D, norm_w, w_out)),
                            dcs, dss, out, batch, d, d_inner, conv_dim, n_heads, d_head, d_state, k, eps, 3)
    for b in range(batch):
        want, wcs, wss = oracle.mamba2_step(x[b, 0], w_in, conv_w, conv_b, dt_bias, a_log, D, norm_w, w_out,
                                            cs[b], ss[b], d, d_inner, conv_dim, n_heads, d_head, d_state, k, eps, 3)
        close(host(out)[b], want, batch, SUM_ORDER)
        close(host(dss)[b], wss, batch, STATE_TOL)
        close(host(dcs)[b], wcs, batch, SUM_ORDER)


@pytest.mark.parametrize("B,T", [(1, 1), (2, 7), (1, 33), (3, 64), (1, 300), (2, 513)])
@pytest.mark.parametrize("wkind", [-2, 2, 3])
def test_forward_sequence(oracle, B, T, wkind):
    """T >= 64 runs the chunked (SSD) scan: 64 = one partial chunk, 300 = two chunks and a
    tail, 513 = four chunks and one step; shorter sequences the sequential scan."""
    from gpu_util import SUM_ORDER, close, dev, empty, fp16_close, host, ops
    c = mamba_case(oracle, B * 1000 + T + wkind, B=B, T=T, d=256, n_heads=4, d_head=64, d_state=128, k=4, wkind=wkind)
    a = c["args"]
    want, want_state = oracle.mamba2_forward(*a, wkind)
    dstate, out = dev(a[9]), empty((B, T, a[12]))
    pw = _dev_params(a[1:9])
    if wkind == -2:
        ops.mamba2_forward(dev(a[0]), *pw, dstate, out, *a[10:])
    else:
        ops.mamba2_forward_half(dev(a[0]), *pw, dstate, out, *a[10:], wkind)
    rows = B * T if wkind != -2 else 1          # fp32 weights never take the tensor-core path
    if wkind == -2 and T >= 64:
        # the chunked scan adds the same fp32 products in another order: bounded against
        # the output scale (elementwise bounds trip on outputs that cancel to ~0)
        fp16_close(host(out), want, frac=1e-4)
        fp16_close(host(dstate), want_state, frac=1e-4)
    else:
        close(host(out), want, rows, dict(rtol=5e-4, atol=5e-5))
        close(host(dstate), want_state, rows, dict(rtol=5e-4, atol=5e-6))


@pytest.mark.parametrize("B,T", [(2, 4096), (1, 4096 + 77), (8, 4096)])
def test_forward_at_the_op_level_benchmark_shape(oracle, B, T):
    """48 heads x 64, d_state 128, 4096 tokens (32 chunks of 128: the state is carried over
    all of them; 4096 + 77 adds a partial tail chunk), Q4_K projections, against the oracle's
    sequential scan (core/mamba_cpu.cpp:81-194).  The model width in front of the projections
    is kept at 256 so the scalar oracle finishes in seconds; conv, scan and gated norm run at
    the full inner width of 3072."""
    from gpu_util import dev, empty, fp16_close, host, ops
    c = mamba_case(oracle, 4000 + B + T, B=B, T=T, d=256, n_heads=48, d_head=64, d_state=128, k=4, wkind=3, w_std=0.1)
    a = c["args"]
    want, want_state = oracle.mamba2_forward(*a, 3)
    dstate, out = dev(a[9]), empty((B, T, a[12]))
    ops.mamba2_forward_half(dev(a[0]), *_dev_params(a[1:9]), dstate, out, *a[10:], 3)
    fp16_close(host(out), want)
    fp16_close(host(dstate), want_state)
    # the tail of the sequence separately: an error in the carried state would show here first
    fp16_close(host(out)[:, -64:], want[:, -64:])


def test_forward_small_state_general_path(oracle):
    """d_state 16 / d_head 32 (shapes outside the register-resident scan's fast cases)."""
    from gpu_util import dev, empty, host, ops
    c = mamba_case(oracle, 77, B=2, T=9, d=64, n_heads=4, d_head=32, d_state=16, k=3, wkind=-2)
    a = c["args"]
    want, want_state = oracle.mamba2_forward(*a, -2)
    dstate, out = dev(a[9]), empty((2, 9, 64))
    ops.mamba2_forward(dev(a[0]), *_dev_params(a[1:9]), dstate, out, *a[10:])
    np.testing.assert_allclose(host(out), want, rtol=5e-4, atol=5e-5)
    np.testing.assert_allclose(host(dstate), want_state, rtol=5e-4, atol=5e-6)


def test_forward_then_steps_continue_state(oracle):
    """A forward over T tokens followed by decode steps equals the oracle doing the same
    (the forward carries the ssm state; its conv window is zero at t = 0 by definition)."""
    from gpu_util import SUM_ORDER, dev, empty, host, ops
    c = mamba_case(oracle, 5, B=1, T=12, d=256, n_heads=4, d_head=64, d_state=128, k=4, wkind=3)
    a = c["args"]
    _, st = oracle.mamba2_forward(*a, 3)
    dstate, out = dev(a[9]), empty((1, 12, 256))
    ops.mamba2_forward_half(dev(a[0]), *_dev_params(a[1:9]), dstate, out, *a[10:], 3)
    np.testing.assert_allclose(host(dstate), st, rtol=5e-4, atol=5e-6)


def test_argument_errors():
    from gpu_util import B200Error, empty, ops
    t = empty(4096)
    with pytest.raises(B200Error, match="n_groups"):
        ops.mamba2_step(t, t, t, t, t, t, t, t, t, t, t, t, 64, 128, 128 + 64, 4, 32, 16, 4, 1e-5)
    with pytest.raises(B200Error, match="unknown qkind"):
        ops.mamba2_step_half(t, t, t, t, t, t, t, t, t, t, t, t, 64, 128, 160, 4, 32, 16, 4, 1e-5, 7)
