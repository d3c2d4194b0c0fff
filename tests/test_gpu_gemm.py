"""GPU parity: the tensor-core (tcgen05) path of the linear layers for many tokens.

Two checks per shape: against the same product computed in fp32 from the
fp16-rounded operands (what the kernel is meant to compute: tight, summation-order
tolerance), and against the CPU oracle on the unrounded activations (the stated
activation bound)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

FP16_OPERANDS = dict(rtol=2e-3, atol=2e-3)


def _fp16_product(x, w16_bits):
    xh = torch.from_numpy(x).cuda().half().float()
    wh = torch.from_numpy(w16_bits.view(np.float16).astype(np.float32)).cuda()
    return (xh.double() @ wh.double().T).float().cpu().numpy()


@pytest.mark.parametrize("M,K,N", [(128, 64, 128), (32, 64, 8), (128, 128, 128), (129, 192, 132), (300, 1536, 200),
                                   (64, 1536, 6448), (1000, 3072, 1536), (2048, 256, 2500)])
def test_linear_fp16_many_tokens(oracle, M, K, N):
    """The last shape has enough tiles for the 256-column store form (ragged last tile)."""
    from gpu_util import ACTIVATION, SUM_ORDER, dev, empty, host, ops
    r = np.random.default_rng(M + K + N)
    x = r.standard_normal((M, K)).astype(np.float32)
    w = oracle.f32_to_f16((r.standard_normal((N, K)) * 0.02).astype(np.float32))
    y = empty((M, N))
    ops.linear_forward_fp16(dev(x), dev(w), y, M, K, N)
    got = host(y)
    np.testing.assert_allclose(got, _fp16_product(x, w), **SUM_ORDER)
    if M * N * K <= 1 << 27:
        np.testing.assert_allclose(got, oracle.linear(x, w, -1, M, K, N), **FP16_OPERANDS)


@pytest.mark.parametrize("kind", [0, 1, 2, 3])
@pytest.mark.parametrize("M,K,N", [(64, 1536, 6448), (257, 512, 1536), (40, 160, 72), (300, 256, 128),
                                   (48, 3072, 256), (33, 1024, 136), (4100, 1024, 2500)])
def test_linear_packed_many_tokens(oracle, kind, M, K, N):
    """K a multiple of 256: weights dequantised inside the GEMM; otherwise (160 for the
    32-weight kinds) through an fp16 copy.  Few output tiles and K >= 512: K is cut
    across CTAs (2, 2, 12 and 4 ways in the cases here) and the partials are added; the
    last shape has enough tiles for the 256-column store form (ragged rows and columns)."""
    if kind == 3 and K % 256:
        pytest.skip("Q4_K rows are multiples of 256 weights")
    from gpu_util import ACTIVATION, SUM_ORDER, dev, empty, fp16_close, host, ops
    r = np.random.default_rng(10 * kind + M)
    x = r.standard_normal((M, K)).astype(np.float32)
    w = oracle.quantize((r.standard_normal(N * K) * 0.02).astype(np.float32), kind)
    y = empty((M, N))
    ops.linear_forward_q4(dev(x), dev(w), y, M, K, N, kind)
    got = host(y)
    w16 = oracle.dequantize(w, N * K, kind).reshape(N, K)          # the fp16-rounded weights
    if kind in (0, 2) or K % 256:
        # the in-kernel expansion is exact for Q4_0 / Q8_0; the fp16-copy path always is
        np.testing.assert_allclose(got, _fp16_product(x, w16), **SUM_ORDER)
    else:
        # Q4_1 / Q4_K inside the GEMM: fp16 FMAs, within one fp16 ulp of the rounded value
        fp16_close(got, _fp16_product(x, w16), frac=1e-3)
    oracle.set_weight_rounding(True)
    try:
        rows = slice(0, min(M, 16))
        want = oracle.linear(x[rows], w, kind, rows.stop, K, N)
    finally:
        oracle.set_weight_rounding(False)
    np.testing.assert_allclose(got[rows], want, **FP16_OPERANDS)


def test_activations_beyond_the_fp16_range_are_clamped(oracle):
    """The tensor-core path rounds its activations to fp16.  Values beyond +-65504 are clamped
    there (pack_rows_f16 and the fp16-row norms), never turned into infinities: the result is
    the product with the clamped activations, finite, and the rows without such values are
    untouched.  (The reference's cuBLAS path converts without a clamp and returns inf / nan
    for such rows, cuda/kernels.cu:104-116; its CPU path computes them in fp32.)"""
    from gpu_util import SUM_ORDER, dev, empty, host, ops
    M, K, N = 64, 512, 256
    r = np.random.default_rng(3)
    x = r.standard_normal((M, K)).astype(np.float32)
    x[5, 7], x[5, 100], x[9, 0] = 1e6, -3e5, 7e4
    w16 = oracle.f32_to_f16((r.standard_normal((N, K)) * 0.02).astype(np.float32))
    wq = oracle.quantize((r.standard_normal(N * K) * 0.02).astype(np.float32), 3)
    clamped = np.clip(x, -65504.0, 65504.0)
    y = empty((M, N))
    ops.linear_forward_fp16(dev(x), dev(w16), y, M, K, N)
    got = host(y)
    assert np.isfinite(got).all()
    np.testing.assert_allclose(got, _fp16_product(clamped, w16), **SUM_ORDER)
    ops.linear_forward_q4(dev(x), dev(wq), y, M, K, N, 3)
    got = host(y)
    assert np.isfinite(got).all()
    from gpu_util import fp16_close
    fp16_close(got, _fp16_product(clamped, oracle.dequantize(wq, N * K, 3).reshape(N, K)), frac=1e-3)


def test_status_word_is_clean_after_gemms():
    """No bounded wait inside the kernels ran out during the tests above."""
    from gpu_util import pkg
    assert pkg.lib().raw("b200_stream_status") == 0
