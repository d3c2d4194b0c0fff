"""Sampling tail on the CPU: the oracle's restatement of core/rng.h and inference/sampler.cpp
against the reference's own objects (where oracle/_ref is built) and against the committed
draws of tests/golden/sampler.npz (made from the reference; make_golden.py sampler)."""
import os

import numpy as np
import pytest

import sampler_cases as sc
from oracle_lib import Sampling

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "sampler.npz")


def test_rng_stream(oracle, ref):
    for seed in (1, 42, 2**63 + 12345):
        assert np.array_equal(oracle.rng_uniform(seed, 500), ref.rng_uniform(seed, 500))


def test_validate(oracle, ref):
    wild = [Sampling(temperature=float("nan"), top_k=-3, top_p=7.0, min_p=1.0, repetition_penalty=-1.0,
                     repetition_window=100000, frequency_penalty=float("inf"), presence_penalty=-9.0, no_repeat_ngram=1),
            Sampling(temperature=9.0, top_k=5000, top_p=-0.5, min_p=float("nan"), repetition_penalty=9.0,
                     repetition_window=-4, frequency_penalty=7.0, presence_penalty=float("nan"), no_repeat_ngram=20)]
    for cfg in wild + list(sc.CONFIGS.values()):
        a, b = oracle.sampling_validate(cfg), ref.sampling_validate(cfg)
        assert np.array_equal(a.f, b.f) and np.array_equal(a.i, b.i)


@pytest.mark.parametrize("name", list(sc.CONFIGS))
def test_sample_matches_the_reference(oracle, ref, name):
    cfg = sc.CONFIGS[name]
    for seed in (1, 2):
        x, h = sc.logits(seed), sc.history(seed)
        assert np.array_equal(oracle.sample(x, h, cfg, 77 + seed, sc.DRAWS), ref.sample(x, h, cfg, 77 + seed, sc.DRAWS)), name
    # an empty history and one shorter than the n-gram
    x = sc.logits(5)
    assert np.array_equal(oracle.sample(x, [], cfg, 9, 8), ref.sample(x, [], cfg, 9, 8))
    assert np.array_equal(oracle.sample(x, [4], cfg, 9, 8), ref.sample(x, [4], cfg, 9, 8))


def test_sample_candidates_matches_the_reference(oracle, ref):
    r = np.random.default_rng(3)
    for K in (1, 2, 40, 128):
        vals = np.sort((r.standard_normal(K) * 3).astype(np.float32))[::-1].copy()
        ids = r.permutation(50000)[:K].astype(np.int32)
        for name in ("default", "hot", "cold", "min_p_only", "temperature_zero"):
            cfg = sc.CONFIGS[name]
            assert np.array_equal(oracle.sample_candidates(vals, ids, cfg, 5, 200), ref.sample_candidates(vals, ids, cfg, 5, 200))
    # degenerate sums: a +inf candidate makes exp(nan) -> the first candidate is returned
    vals = np.array([np.inf, 1.0, 0.0], np.float32)
    ids = np.array([7, 8, 9], np.int32)
    assert np.array_equal(oracle.sample_candidates(vals, ids, sc.CONFIGS["hot"], 5, 4),
                          ref.sample_candidates(vals, ids, sc.CONFIGS["hot"], 5, 4))


def test_draws_follow_the_distribution(oracle):
    """20000 draws from 4 candidates: frequencies within 4 sigma of the softmax."""
    vals = np.array([2.0, 1.0, 0.5, -1.0], np.float32)
    ids = np.arange(4, dtype=np.int32)
    cfg = Sampling(temperature=1.0, top_k=4, top_p=1.0, min_p=0.0)
    got = np.bincount(oracle.sample_candidates(vals, ids, cfg, 11, 20000), minlength=4) / 20000
    p = np.exp(vals - vals.max())
    p /= p.sum()
    assert np.all(np.abs(got - p) < 4 * np.sqrt(p * (1 - p) / 20000))


def test_cross_entropy_matches_the_reference(oracle, ref):
    r = np.random.default_rng(8)
    x = (r.standard_normal((37, 1000)) * 3).astype(np.float32)
    t = r.integers(0, 1000, 37).astype(np.int32)
    t[[3, 9]] = -100
    for z in (0.0, 1e-4):
        (a, na), (b, nb) = oracle.cross_entropy(x, t, z), ref.cross_entropy(x, t, z)
        assert na == nb == 35
        assert abs(a - b) <= 1e-9 * abs(b)        # the reference sums rows under OpenMP: order only


def test_golden_draws(oracle):
    """The committed draws of the reference's Sampler."""
    g = np.load(GOLD)
    for name, cfg in sc.CONFIGS.items():
        for seed in (1, 2):
            want = g[f"{name}/{seed}"]
            assert np.array_equal(oracle.sample(sc.logits(seed), sc.history(seed), cfg, 77 + seed, sc.DRAWS), want), name
    assert np.array_equal(oracle.rng_uniform(42, 500), g["uniform/42"])
    total, count = oracle.cross_entropy(sc.logits(3, 4000).reshape(4, 1000), g["ce/targets"], 1e-4)
    assert count == int(g["ce/count"]) and abs(total - float(g["ce/sum"])) <= 1e-9 * abs(total)
