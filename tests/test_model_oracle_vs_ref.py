"""Pins the model-level oracle (the Python walk of the reference's per-token op
sequence over the scalar oracle) to the reference's own Model + Generator on its
CPU device, on the same seeded weights: logits must agree to summation-order noise
and the greedy picks must be identical."""
import numpy as np
import pytest

from model_util import TINY, OracleDecoder, RefGenerator, model_from_f32, random_f32_params
from oracle_lib import Ref


@pytest.mark.skipif(not Ref.available(), reason="oracle/_ref not built (reference sources not mounted)")
@pytest.mark.parametrize("qkind", [2, 0])
def test_decoder_matches_reference_generator(oracle, qkind):
    cfg = dict(TINY, qkind=qkind, hidden=128, mamba_heads=4, mamba_d_head=64, n_heads=2, n_kv=1, expert_dim=64,
               shared_dim=64, vocab=256, mamba_d_state=64)
    params = random_f32_params(cfg, seed=3)
    ref = RefGenerator(cfg, params, max_ctx=16)
    ora = OracleDecoder(oracle, model_from_f32(oracle, cfg, params), max_ctx=16)
    r = np.random.default_rng(1)
    tok = 5
    for s in range(10):
        a, b = ora.step(tok), ref.step(tok)
        np.testing.assert_allclose(a, b, rtol=2e-4, atol=2e-5)
        assert int(np.argmax(a)) == int(np.argmax(b))
        tok = int(r.integers(0, cfg["vocab"])) if s < 5 else int(np.argmax(b))
    ref.close()


def oracle_score(oracle, ora, tokens, mask=None):
    """Generator::score_tokens over the stepwise oracle: position i is scored against token
    i + 1 when that token is supervised; the cross-entropy in double (core/math_cpu.cpp:560)."""
    tokens = np.asarray(tokens, np.int32)
    logits = np.stack([ora.step(int(t)) for t in tokens[:-1]])
    targets = tokens[1:].copy()
    if mask is not None:
        targets[np.asarray(mask)[1:] == 0] = -100
    total, n = oracle.cross_entropy(logits, targets)
    return (total / n if n else 0.0), n


@pytest.mark.skipif(not Ref.available(), reason="oracle/_ref not built (reference sources not mounted)")
def test_score_tokens_matches_reference_generator(oracle):
    cfg = dict(TINY, qkind=2, hidden=128, mamba_heads=4, mamba_d_head=64, n_heads=2, n_kv=1, expert_dim=64,
               shared_dim=64, vocab=256, mamba_d_state=64)
    params = random_f32_params(cfg, seed=4)
    ref = RefGenerator(cfg, params, max_ctx=64)
    ora = OracleDecoder(oracle, model_from_f32(oracle, cfg, params), max_ctx=64)
    tokens = np.random.default_rng(2).integers(0, cfg["vocab"], 24).astype(np.int32)
    a, na = oracle_score(oracle, ora, tokens)
    b, nb = ref.score_tokens(tokens)
    assert na == nb == 23
    assert abs(a - b) < 2e-4 * abs(b)
    mask = np.ones(24, np.uint8)
    mask[3:9] = 0
    ora.reset()
    a, na = oracle_score(oracle, ora, tokens, mask)
    b, nb = ref.score_tokens(tokens, mask)
    assert na == nb == 17
    assert abs(a - b) < 2e-4 * abs(b)
    ref.close()
