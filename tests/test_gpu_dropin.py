"""The drop-in itself: the reference engine's unmodified Model + Generator +
KVCache, compiled for its CUDA device and linked against this repository's shim and
libb200ops instead of its own CUDA library (oracle/_ref/libgai_b200.so), against the
same engine on its CPU device, teacher-forced on identical seeded weights."""
import os

import numpy as np
import pytest

from model_util import CONFIG_1, TINY, RefGenerator, random_f32_params
from oracle_lib import ROOT

pytestmark = pytest.mark.gpu
B200_SO = os.path.join(ROOT, "oracle", "_ref", "libgai_b200.so")
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libgai_ref.so")
needs_ref = pytest.mark.skipif(not (os.path.exists(B200_SO) and os.path.exists(REF_SO)),
                               reason="oracle/_ref libraries not built (reference sources were not mounted)")


def _run(cfg, steps, seed):
    params = random_f32_params(cfg, seed=seed)
    cpu = RefGenerator(cfg, params, max_ctx=steps + 2, lib="ref")
    gpu = RefGenerator(cfg, params, max_ctx=steps + 2, lib="b200")
    r = np.random.default_rng(seed + 1)
    tok, agree, worst = 7, 0, 0.0
    for s in range(steps):
        want, got = cpu.step(tok), gpu.step(tok)
        err = np.abs(got - want)
        worst = max(worst, float(err.max()))
        assert np.all(err <= 2e-2 + 1e-2 * np.abs(want)), f"step {s}: max abs err {err.max()}"
        agree += int(np.argmax(got) == np.argmax(want))
        tok = int(r.integers(0, cfg["vocab"])) if s < steps // 2 else int(np.argmax(want))
    cpu.close()
    gpu.close()
    return agree / steps, worst


@needs_ref
@pytest.mark.parametrize("qkind", [2, 0, 1])
def test_reference_generator_on_b200_backend_tiny(qkind):
    cfg = dict(TINY, qkind=qkind, mamba_d_state=64)
    rate, worst = _run(cfg, steps=16, seed=11)
    assert rate >= 0.99 and worst < 2e-3


@needs_ref
def test_reference_generator_on_b200_backend_config1():
    """Config 1 (hidden 768, 8 layers, 16 experts top-2, Q8_0, RoPE) at a reduced vocabulary."""
    cfg = dict(CONFIG_1, vocab=4096)
    rate, worst = _run(cfg, steps=24, seed=0)
    assert rate >= 0.99 and worst < 2e-3
