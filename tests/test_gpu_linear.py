"""GPU parity: dequantiser (bit-exact) and the linear layers, through the C ABI."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _w(oracle, r, N, K, kind):
    return oracle.quantize((r.standard_normal(N * K) * 0.02).astype(np.float32), kind)


@pytest.mark.parametrize("kind", [0, 1, 2, 3])
@pytest.mark.parametrize("n", [256 * 3, 256 * 1027])
def test_dequantize_bit_exact(oracle, kind, n):
    from gpu_util import dev, empty, host, ops
    r = np.random.default_rng(kind * 7 + 1)
    x = (r.standard_normal(n) * 0.02).astype(np.float32)
    x[:256] = 0.0
    packed = oracle.quantize(x, kind)
    want = oracle.dequantize(packed, n, kind)
    got = empty(n, torch.int16)
    ops.dequantize_quant(dev(packed), got, n, kind)
    assert np.array_equal(host(got, np.uint16), want)
    # ragged element count (n not a multiple of 8): only the first m values are written
    m = n - 37
    got2 = empty(n, torch.int16)
    ops.dequantize_quant(dev(packed), got2, m, kind)
    assert np.array_equal(host(got2, np.uint16)[:m], want[:m])
    assert (host(got2)[m:] == -7).all()


@pytest.mark.parametrize("kind", [0, 1, 2, 3])
def test_dequantize_random_bytes(oracle, kind):
    """Any byte pattern (all scale codes, negative/denormal fp16 scales) decodes identically."""
    from gpu_util import dev, empty, host, ops
    from oracle_lib import BLOCK_BYTES, BLOCK_ELEMS
    r = np.random.default_rng(99 + kind)
    nb = 4096
    packed = r.integers(0, 256, nb * BLOCK_BYTES[kind], dtype=np.uint8)
    # keep fp16 headers finite so NaN payloads do not enter the comparison
    blk = packed.reshape(nb, BLOCK_BYTES[kind])
    blk[:, 1] &= 0x7B
    if kind in (1, 3):
        blk[:, 3] &= 0x7B
    n = nb * BLOCK_ELEMS[kind]
    want = oracle.dequantize(packed, n, kind)
    got = empty(n, torch.int16)
    ops.dequantize_quant(dev(packed), got, n, kind)
    assert np.array_equal(host(got, np.uint16), want)


def _check_packed(oracle, got, x, w, kind, M, K, N):
    """Packed-weight linears: tight against the product of the exact dequantised values
    (what the reference's fused CUDA kernel computes); within the stated activation
    tolerance of the reference's CPU path, which rounds every dequantised weight through
    fp16 first (core/ops.cpp:392) - a 2^-12 relative perturbation per weight."""
    from gpu_util import ACTIVATION, SUM_ORDER, close
    close(got, oracle.linear_exact(x, w, kind, M, K, N), M, SUM_ORDER)
    oracle.set_weight_rounding(True)
    rounded = oracle.linear(x, w, kind, M, K, N)
    oracle.set_weight_rounding(False)
    np.testing.assert_allclose(got, rounded, **ACTIVATION)
    assert np.abs(got - rounded).max() <= 2e-3 * max(1.0, np.abs(rounded).max())


SHAPES = [  # (K, N): config-1 and H-Tiny projections, scaled-down vocab
    (768, 3224), (1536, 768), (1536, 6448), (3072, 1536), (512, 1536), (1024, 1536), (256, 40),
]


@pytest.mark.parametrize("kind", [0, 1, 2, 3])
@pytest.mark.parametrize("K,N", SHAPES)
def test_linear_q4_decode(oracle, kind, K, N):
    from gpu_util import SUM_ORDER, dev, empty, host, ops
    if kind == 3 and K % 256:
        pytest.skip("Q4_K needs K % 256 == 0")
    r = np.random.default_rng(K + N + kind)
    w = _w(oracle, r, N, K, kind)
    x = r.standard_normal((1, K)).astype(np.float32)
    y = empty((1, N))
    ops.linear_forward_q4(dev(x), dev(w), y, 1, K, N, kind)
    _check_packed(oracle, host(y), x, w, kind, 1, K, N)


@pytest.mark.parametrize("kind", [2, 3])
@pytest.mark.parametrize("M", [2, 3, 4, 7, 8, 9, 64])
def test_linear_q4_batched(oracle, kind, M):
    from gpu_util import SUM_ORDER, dev, empty, host, ops
    K, N = 512, 200
    r = np.random.default_rng(M * 3 + kind)
    w = _w(oracle, r, N, K, kind)
    x = r.standard_normal((M, K)).astype(np.float32)
    y = empty((M, N))
    ops.linear_forward_q4(dev(x), dev(w), y, M, K, N, kind)
    _check_packed(oracle, host(y), x, w, kind, M, K, N)


@pytest.mark.parametrize("M,K,N", [(1, 1536, 4096), (5, 768, 300), (2, 100, 7), (1, 36, 3)])
def test_linear_fp16_and_fp32(oracle, M, K, N):
    from gpu_util import SUM_ORDER, dev, empty, host, ops
    r = np.random.default_rng(M + K + N)
    x = r.standard_normal((M, K)).astype(np.float32)
    wf = (r.standard_normal((N, K)) * 0.05).astype(np.float32)
    wh = oracle.f32_to_f16(wf)
    y = empty((M, N))
    ops.linear_forward_fp16(dev(x), dev(wh), y, M, K, N)
    np.testing.assert_allclose(host(y), oracle.linear(x, wh, -1, M, K, N), **SUM_ORDER)
    for fn in (ops.linear_forward, ops.linear_forward_f32):
        y = empty((M, N))
        fn(dev(x), dev(wf), y, M, K, N)
        np.testing.assert_allclose(host(y), oracle.linear(x, wf, -2, M, K, N), **SUM_ORDER)
    y = empty((M, N))
    ops.gemm(0, 1, M, N, K, 1.0, dev(x), K, dev(wf), K, 0.0, y, N)
    np.testing.assert_allclose(host(y), oracle.linear(x, wf, -2, M, K, N), **SUM_ORDER)


def test_linear_argument_errors(oracle):
    from gpu_util import B200Error, empty, ops
    x, w, y = empty((1, 48)), empty(64, torch.uint8), empty((1, 2))
    with pytest.raises(B200Error, match="multiple of 32"):
        ops.linear_forward_q4(x, w, y, 1, 48, 2, 2)           # K % 32 != 0 (core/ops.cpp:369)
    with pytest.raises(B200Error, match="multiple of 256"):
        ops.linear_forward_q4(x, w, y, 1, 32, 2, 3)
    with pytest.raises(B200Error, match="unknown kind"):
        ops.linear_forward_q4(x, w, y, 1, 32, 2, 9)
    ops.linear_forward_q4(x, w, y, 0, 32, 2, 2)                # M == 0 returns silently (ops.cpp:362)
    with pytest.raises(B200Error):
        ops.gemm(1, 0, 2, 2, 2, 1.0, x, 2, x, 2, 0.0, y, 2)   # training-form GEMM is not provided


def test_linear_linearity_full_size(oracle):
    """H-Tiny in_proj at full size: W(x1 + 2 x2) == W x1 + 2 W x2 up to rounding."""
    from gpu_util import dev, empty, host, ops
    K, N = 1536, 6448
    r = np.random.default_rng(5)
    w = dev(r.integers(0, 256, N * K // 256 * 144, dtype=np.uint8))
    # plausible fp16 scales: clear sign/exponent top bits of d and dmin
    wv = w.view(-1, 144)
    wv[:, 1] = 0x1C
    wv[:, 3] = 0x1C
    x1 = r.standard_normal((1, K)).astype(np.float32)
    x2 = r.standard_normal((1, K)).astype(np.float32)
    ys = []
    for x in (x1, x2, x1 + 2 * x2):
        y = empty((1, N))
        ops.linear_forward_q4(dev(x), w, y, 1, K, N, 3)
        ys.append(host(y).astype(np.float64))
    scale = np.abs(ys[2]).max()
    assert np.abs(ys[0] + 2 * ys[1] - ys[2]).max() <= 1e-5 * scale


def test_converts_and_split(oracle):
    from gpu_util import dev, empty, host, ops
    r = np.random.default_rng(11)
    x = (r.standard_normal(5000) * np.exp(r.uniform(-12, 8, 5000))).astype(np.float32)
    h = empty(5000, torch.int16)
    ops.convert_f32_to_f16(dev(x), h, 5000)
    assert np.array_equal(host(h, np.uint16), oracle.f32_to_f16(x))
    back = empty(5000)
    ops.convert_f16_to_f32(h, back, 5000)
    assert np.array_equal(host(back), oracle.f16_to_f32(host(h, np.uint16)))
    qkv = r.standard_normal((3, 20)).astype(np.float32)
    q, k, v = empty((3, 12)), empty((3, 4)), empty((3, 4))
    ops.split_qkv(dev(qkv), q, k, v, 3, 12, 4)
    assert np.array_equal(host(q), qkv[:, :12]) and np.array_equal(host(k), qkv[:, 12:16])
    assert np.array_equal(host(v), qkv[:, 16:])
