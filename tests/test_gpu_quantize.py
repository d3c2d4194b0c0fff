"""GPU parity: device quantisers are bit-identical to the CPU functions."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind", [0, 1, 2, 3, 4])
def test_quantize_bit_exact(oracle, kind):
    from gpu_util import dev, empty, host, pkg
    from oracle_lib import packed_bytes
    r = np.random.default_rng(kind)
    n = 256 * 4099
    x = (r.standard_normal(n) * 0.02).astype(np.float32)
    x[:256] = 0.0                                  # zero block
    x[256:512] = np.abs(x[256:512])                # all-positive block (Q4_K min = 0)
    x[512:768] = 0.5                               # constant block (zero range)
    x[1024 + 7] = np.inf                           # non-finite -> zero block
    x[2048:2304] *= 1e-6
    x[4096 + 3] = np.nan                           # zero block; kind 4: the element's code is 0
    x[8192:8448] = -np.abs(x[8192:8448])           # all negative (kind 4: positive scale)
    x[8448:8480] = np.float32(-0.125)              # every element the extreme
    want = oracle.quantize(x, kind)
    out = empty(packed_bytes(kind, n), torch.uint8)
    pkg.lib().b200_quantize(dev(x), out, n, kind)
    got = host(out)
    bad = np.flatnonzero(got != want)
    assert bad.size == 0, f"{bad.size} bytes differ, first at {bad[:5]}"


def test_quantize_roundtrip_full_size(oracle):
    """One H-Tiny expert tensor (64 x 512 x 1536): quantise on the device, dequantise on
    the device, error bounded by half a quantisation step per 32-weight sub-block."""
    from gpu_util import empty, host, pkg, ops
    from oracle_lib import packed_bytes
    n = 64 * 512 * 1536
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(n, device="cuda", generator=g) * 0.02
    packed = empty(packed_bytes(3, n), torch.uint8)
    pkg.lib().b200_quantize(x, packed, n, 3)
    back = empty(n, torch.int16)
    ops.dequantize_quant(packed, back, n, 3)
    y = back.view(torch.float16).float()
    # per 256-weight super-block: nibble rounding (half a step) plus the 6-bit rounding of
    # the sub-block scale (15 codes x 1/126 of the largest step) and of the minimum
    xs, ys = x.view(-1, 8, 32), y.view(-1, 8, 32)
    lo = xs.min(2).values.clamp(max=0)
    step = (xs.max(2).values - lo) / 15
    bound = 0.5 * step.max(1).values + 15.0 / 126 * step.max(1).values + (-lo).max(1).values / 126 + 1e-4
    err = (xs - ys).abs().amax((1, 2))
    assert bool((err <= bound * 1.05).all())
    assert float((xs - ys).abs().mean()) < 1.5e-3


def test_quantize_rejects_misaligned_buffers():
    from gpu_util import B200Error, empty, pkg
    x = torch.zeros(1024 + 1, device="cuda")
    out = empty(2048, torch.uint8)
    with pytest.raises(B200Error):
        pkg.lib().b200_quantize(x[1:], out, 1024, 2)          # source not 16-byte aligned
    with pytest.raises(B200Error):
        pkg.lib().b200_quantize(x, out, 1000, 2)              # not whole blocks
    with pytest.raises(B200Error):
        pkg.lib().b200_quantize(x, out, 1024, 7)              # unknown kind
