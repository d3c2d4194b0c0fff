"""Sampling configurations and inputs shared by the oracle-vs-reference pin, the golden
fixture tests/golden/sampler.npz (tests/golden/make_golden.py sampler) and the GPU tests."""
import numpy as np

from oracle_lib import Sampling

VOCAB = 3000
# name -> SamplingConfig; together they reach every branch of Sampler::sample
CONFIGS = {
    "default": Sampling(),                                                        # top-k 40, top-p .92, min-p .05, rep 1.12
    "hot": Sampling(temperature=1.7, top_k=200, top_p=0.99, min_p=0.0, repetition_penalty=1.0),
    "top_p_only": Sampling(temperature=1.0, top_k=0, top_p=0.6, min_p=0.0, repetition_penalty=1.0),
    "min_p_only": Sampling(temperature=1.2, top_k=0, top_p=1.0, min_p=0.2, repetition_penalty=1.0),
    "no_filter": Sampling(temperature=0.9, top_k=0, top_p=1.0, min_p=0.0, repetition_penalty=1.3, frequency_penalty=0.2,
                          presence_penalty=0.1, repetition_window=0),
    "ngram": Sampling(temperature=0.7, top_k=5, top_p=1.0, min_p=0.0, no_repeat_ngram=3, repetition_window=16),
    "greedy": Sampling(greedy=True),
    "temperature_zero": Sampling(temperature=0.0, repetition_penalty=1.5),
    "top_k_one": Sampling(top_k=1),
    "cold": Sampling(temperature=0.05, top_k=50, top_p=0.5, min_p=0.0),
}
DRAWS = 64


def logits(seed=0, vocab=VOCAB):
    r = np.random.default_rng(seed)
    x = (r.standard_normal(vocab) * 2.5).astype(np.float32)
    x[r.integers(0, vocab, 8)] += 6.0        # a few clear favourites
    return x


def history(seed=0, n=200, vocab=VOCAB):
    r = np.random.default_rng(100 + seed)
    h = r.integers(0, vocab, n).astype(np.int32)
    h[::7] = h[0]                            # repeats (frequency counts > 1)
    h[-2:] = h[10:12]                        # the last bigram occurred before: an n-gram ban applies
    h[5] = -1                                # out-of-range ids are skipped
    h[6] = vocab + 3
    return h
