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


@needs_ref
@pytest.mark.parametrize("qkind", [2, 0])
def test_reference_score_tokens_on_b200_backend(qkind):
    """Generator::score_tokens (inference/generator.cpp:1217-1294), unmodified, on this backend: its
    Model::forward runs every layer through the many-token ops of the shim and the loss through
    b200_softmax_cross_entropy (cuda_ops.h:278 with a null gradient buffer); compared with the same
    engine on its CPU device - with and without a supervision mask."""
    cfg = dict(TINY, qkind=qkind, hidden=256, vocab=512)
    params = random_f32_params(cfg, seed=4)
    tokens = np.random.default_rng(2).integers(0, cfg["vocab"], 80).astype(np.int32)
    mask = np.ones(80, np.uint8)
    mask[10:25] = 0
    cpu = RefGenerator(cfg, params, max_ctx=128, lib="ref")
    gpu = RefGenerator(cfg, params, max_ctx=128, lib="b200")
    for m in (None, mask):
        (want, n_want), (got, n_got) = cpu.score_tokens(tokens, m), gpu.score_tokens(tokens, m)
        assert n_got == n_want == (79 if m is None else 64)
        assert abs(got - want) <= 1e-3 * abs(want), (got, want)
    cpu.close()
    gpu.close()


def _common_prefix(a, b):
    n = min(len(a), len(b))
    return int(np.argmax(np.append(a[:n] != b[:n], True)))


@needs_ref
def test_reference_penalised_greedy_generation_on_b200_backend():
    """Generator::generate, unmodified, greedy with all three penalties: on its CUDA device (this
    backend) the engine takes its fast path (inference/generator.cpp:1036-1047) - it hands
    b200_apply_rep_penalties the window of its HOST history and takes b200_argmax_token of the
    penalised device logits - while on its CPU device Sampler::sample does both on the host."""
    from oracle_lib import Sampling
    cfg = dict(TINY, qkind=2, vocab=1024)            # the fast path needs a vocabulary of 512 or more
    params = random_f32_params(cfg, seed=6)
    sampling = Sampling(temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, repetition_penalty=1.3, repetition_window=16,
                        frequency_penalty=0.2, presence_penalty=0.1, greedy=True)
    cpu = RefGenerator(cfg, params, max_ctx=128, lib="ref")
    gpu = RefGenerator(cfg, params, max_ctx=128, lib="b200")
    commons = []
    for p in range(3):      # a free-running generation stays equal until the first near-tie: three prompts, the median counts
        prompt = np.random.default_rng(3 + p).integers(0, cfg["vocab"], 12).astype(np.int32)
        want = cpu.generate(prompt, 48, sampling, seed=1)
        got = gpu.generate(prompt, 48, sampling, seed=1)
        assert len(want) == len(got) == 48
        commons.append(_common_prefix(want, got))
    cpu.close()
    gpu.close()
    print("common prefixes", commons)
    assert sorted(commons)[1] >= 40, commons


@needs_ref
def test_reference_sampled_generation_on_b200_backend():
    """Generator::generate with sampling, unmodified: the fast path applies the penalties and
    b200_topk_select on the device, copies the K candidates to the host and draws with
    Sampler::sample_candidates there (inference/generator.cpp:1047-1056); on the CPU device
    Sampler::sample works on the full logits.  Same seed, same draws: the generations agree until a
    draw falls within the logits' tolerance of a boundary between two candidates (a first
    difference changes everything after it), so the bar is on the common prefixes of several
    seeds, not on equality of the whole."""
    from oracle_lib import Sampling
    cfg = dict(TINY, qkind=2, vocab=1024)
    params = random_f32_params(cfg, seed=6)
    prompt = np.random.default_rng(3).integers(0, cfg["vocab"], 12).astype(np.int32)
    sampling = Sampling(temperature=0.9, top_k=8, top_p=0.95, min_p=0.0, repetition_penalty=1.2, repetition_window=16)
    cpu = RefGenerator(cfg, params, max_ctx=256, lib="ref")
    gpu = RefGenerator(cfg, params, max_ctx=256, lib="b200")
    commons = []
    for seed in (123, 124, 125, 126):
        want = cpu.generate(prompt, 32, sampling, seed=seed)
        got = gpu.generate(prompt, 32, sampling, seed=seed)
        assert len(want) == len(got) == 32
        commons.append(_common_prefix(want, got))
    cpu.close()
    gpu.close()
    print("common prefixes", commons)
    assert sorted(commons)[1] >= 12 and sum(commons) >= 0.5 * 4 * 32, commons
