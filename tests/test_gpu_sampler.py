"""GPU parity of the sampling tail: the device generator, Sampler::sample_candidates,
Sampler::sample, the cross-entropy and the decoder's sampled loop / perplexity scoring against
the CPU oracle (itself pinned to the reference's Sampler: tests/test_sampler_oracle.py) and
against the reference's own committed draws (tests/golden/sampler.npz).

Picks are integers and must be identical.  (The device's exp() in double may differ from the
host's in the last bit; a pick could only change if the uniform draw fell within ~1e-16 of a
boundary of the cumulative distribution.)
"""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import sampler_cases as sc
from model_util import TINY, B200Sampling, CudaDecoder, OracleDecoder, cached_model
from oracle_lib import Sampling

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "sampler.npz"))


def _states(lib, seed, rows):
    st = torch.zeros(rows * 4, dtype=torch.int64, device="cuda")
    lib.b200_rng_seed(seed, st, rows)
    return st


def test_rng_stream(oracle):
    from gpu_util import empty, host, pkg
    lib = pkg.lib()
    st = _states(lib, 42, 3)
    out = empty(500)
    lib.b200_rng_uniform(st, out, 500)
    assert np.array_equal(host(out), GOLD["uniform/42"])
    # stream i is Rng(seed + i)
    states = host(st).view(np.uint64).reshape(3, 4)
    assert np.array_equal(states[1], oracle.rng_state(43)) and np.array_equal(states[2], oracle.rng_state(44))
    lib.b200_rng_uniform(st, out, 7)                       # the state went on
    assert np.array_equal(host(out)[:7], oracle.rng_uniform(42, 507)[500:])


def test_validate_matches(oracle):
    from gpu_util import pkg
    wild = [Sampling(temperature=float("nan"), top_k=-3, top_p=7.0, min_p=1.0, repetition_penalty=-1.0,
                     repetition_window=100000, frequency_penalty=float("inf"), presence_penalty=-9.0, no_repeat_ngram=1),
            Sampling(temperature=9.0, top_k=5000, top_p=-0.5, min_p=float("nan"), repetition_penalty=9.0,
                     repetition_window=-4, frequency_penalty=7.0, presence_penalty=float("nan"), no_repeat_ngram=20)]
    for cfg in wild + list(sc.CONFIGS.values()):
        s = B200Sampling.of(cfg, 1)
        pkg.lib().b200_sampling_validate(C.byref(s))
        want = oracle.sampling_validate(cfg)
        got_f = np.array([s.temperature, s.top_p, s.min_p, s.repetition_penalty, s.frequency_penalty, s.presence_penalty],
                         np.float32)
        assert np.array_equal(got_f, want.f)
        assert [s.top_k, s.repetition_window, s.no_repeat_ngram, s.greedy] == want.i.tolist()


@pytest.mark.parametrize("K", [1, 2, 40, 128, 1000, 2048])
def test_sample_candidates(oracle, K):
    from gpu_util import dev, empty, host, pkg
    lib = pkg.lib()
    r = np.random.default_rng(K)
    rows, draws = 3, 40
    vals = (r.standard_normal((rows, K)) * 3).astype(np.float32)
    ids = np.stack([r.permutation(100352)[:K] for _ in range(rows)]).astype(np.int32)
    if K >= 40:
        vals[0, 5] = vals[0, 17]                    # equal values: the lower id comes first
    dv, di = dev(vals), dev(ids)
    for name in ("default", "hot", "cold", "min_p_only", "top_p_only", "temperature_zero"):
        cfg = oracle.sampling_validate(sc.CONFIGS[name])
        st = _states(lib, 900, rows)
        want_states = [oracle.rng_state(900 + i) for i in range(rows)]
        nxt = empty(rows, torch.int32)
        s = B200Sampling.of(cfg)
        for _ in range(draws):
            lib.b200_sample_candidates(dv, di, K, rows, C.byref(s), st, nxt)
            got = host(nxt)
            want = [oracle.candidates_with_state(vals[i], ids[i], cfg, want_states[i]) for i in range(rows)]
            assert got.tolist() == want, name
        assert np.array_equal(host(st).view(np.uint64).reshape(rows, 4), np.stack(want_states)), name


@pytest.mark.parametrize("name", list(sc.CONFIGS))
def test_sample_logits_reproduces_the_reference_draws(oracle, name):
    """Row 0 / row 1 = the two committed cases of the reference's Sampler (seeds 78 and 79 are
    Rng(78 + row)); row 2 has no usable history."""
    from gpu_util import dev, empty, host, pkg
    lib = pkg.lib()
    cfg = sc.CONFIGS[name]
    logits = np.stack([sc.logits(1), sc.logits(2), sc.logits(3)])
    hist = np.zeros((3, 256), np.int32)
    hist[0, :200], hist[1, :200] = sc.history(1), sc.history(2)
    lens = np.array([200, 200, 0], np.int32)
    dh, dl = dev(hist), dev(lens)
    st = _states(lib, 78, 3)
    state2 = oracle.rng_state(80)
    ocfg = oracle.sampling_validate(cfg)
    nxt = empty(3, torch.int32)
    got = np.zeros((sc.DRAWS, 3), np.int32)
    s = B200Sampling.of(cfg)
    for i in range(sc.DRAWS):
        work = dev(logits)                          # fresh logits per draw, as the fixture's generator did
        lib.b200_sample_logits(work, sc.VOCAB, 3, dh, 256, dl, C.byref(s), st, nxt)
        got[i] = host(nxt)
        assert got[i, 2] == oracle.sample_with_state(logits[2].copy(), [], ocfg, state2)
    assert np.array_equal(got[:, 0], GOLD[f"{name}/1"]), name
    assert np.array_equal(got[:, 1], GOLD[f"{name}/2"]), name


def test_sample_logits_full_vocabulary(oracle):
    """H-Tiny's vocabulary: the K-pass selection (top-k 40), the full sort (top-k 300 and
    top-p without top-k) and the unfiltered draw."""
    from gpu_util import dev, empty, host, pkg
    lib = pkg.lib()
    V = 100352
    logits = np.stack([sc.logits(10, V), sc.logits(11, V)])
    hist = np.stack([sc.history(10, 2000, V), sc.history(11, 2000, V)])
    dh, dl = dev(hist), dev(np.array([2000, 1500], np.int32))
    for cfg in (Sampling(), Sampling(top_k=300, top_p=0.95, min_p=0.0), Sampling(top_k=0, top_p=0.9, min_p=0.0, temperature=1.3),
                Sampling(top_k=0, top_p=1.0, min_p=0.0, temperature=1.0, repetition_window=0)):
        st = _states(lib, 5, 2)
        states = [oracle.rng_state(5), oracle.rng_state(6)]
        nxt = empty(2, torch.int32)
        s = B200Sampling.of(cfg)
        for _ in range(6):
            work = dev(logits)
            lib.b200_sample_logits(work, V, 2, dh, 2000, dl, C.byref(s), st, nxt)
            want = [oracle.sample_with_state(logits[0].copy(), hist[0], cfg, states[0]),
                    oracle.sample_with_state(logits[1].copy(), hist[1, :1500], cfg, states[1])]
            assert host(nxt).tolist() == want


def test_penalties_and_ban_leave_the_reference_logits(oracle):
    from gpu_util import dev, host, empty, pkg
    cfg = Sampling(greedy=True, repetition_penalty=1.3, frequency_penalty=0.2, presence_penalty=0.1, repetition_window=64,
                   no_repeat_ngram=3)
    x, h = sc.logits(4), sc.history(4)
    want = x.copy()
    tok = oracle.sample_with_state(want, h, cfg, oracle.rng_state(1))
    work = dev(x)
    nxt = empty(1, torch.int32)
    st = _states(pkg.lib(), 1, 1)
    pkg.lib().b200_sample_logits(work, sc.VOCAB, 1, dev(h), h.size, dev(np.array([h.size], np.int32)),
                                 C.byref(B200Sampling.of(cfg)), st, nxt)
    assert np.array_equal(host(work).view(np.uint32), want.view(np.uint32))
    assert int(host(nxt)[0]) == tok
    assert np.array_equal(host(st).view(np.uint64), oracle.rng_state(1))     # greedy draws nothing


def test_cross_entropy(oracle):
    from gpu_util import B200Error, dev, pkg
    lib = pkg.lib()
    t4 = GOLD["ce/targets"]
    total, count = C.c_double(), C.c_int64()
    lib.b200_softmax_cross_entropy(dev(sc.logits(3, 4000)), dev(t4), None, 4, 1000, C.byref(total), C.byref(count),
                                   C.c_float(1e-4))
    assert count.value == int(GOLD["ce/count"]) and abs(total.value - float(GOLD["ce/sum"])) <= 1e-9 * abs(total.value)
    r = np.random.default_rng(3)
    V, n = 100352, 9
    x = (r.standard_normal((n, V)) * 2).astype(np.float32)
    t = r.integers(0, V, n).astype(np.int32)
    t[4] = -100
    lib.b200_softmax_cross_entropy(dev(x), dev(t), None, n, V, C.byref(total), C.byref(count), C.c_float(0.0))
    want, nw = oracle.cross_entropy(x, t)
    assert count.value == nw == 8 and abs(total.value - want) <= 1e-9 * abs(want)
    t[2] = V
    with pytest.raises(B200Error):
        lib.b200_softmax_cross_entropy(dev(x), dev(t), None, n, V, C.byref(total), C.byref(count), C.c_float(0.0))
    with pytest.raises(B200Error):                      # the gradient is a training op
        lib.b200_softmax_cross_entropy(dev(x), dev(t), dev(x), n, V, C.byref(total), C.byref(count), C.c_float(0.0))


@pytest.mark.parametrize("mode", [(0, 0), (1, 1), (2, 1)])
def test_decoder_samples_like_the_host_loop(oracle, mode):
    """A sampled generation on the device (history, penalties, selection and generator state all
    resident) against Sampler::sample applied on the host to the same logits: a second, greedy
    decoder fed the same tokens supplies the logits before penalties."""
    model = cached_model(oracle, TINY, seed=2)
    V = TINY["vocab"]
    cfg = oracle.sampling_validate(Sampling(temperature=1.1, top_k=20, top_p=0.9, min_p=0.02, repetition_penalty=1.3,
                                            repetition_window=8, frequency_penalty=0.1))
    sampled = CudaDecoder(model, batch=2, max_ctx=64) if mode[0] < 2 else CudaDecoder(model, batch=1, max_ctx=64)
    B = sampled.batch
    plain = CudaDecoder(model, batch=B, max_ctx=64)
    sampled.configure(*mode)
    plain.configure(1, 0)
    sampled.set_sampling(cfg, seed=33)
    states = [oracle.rng_state(33 + b) for b in range(B)]
    prompt = np.random.default_rng(5).integers(0, V, (B, 9)).astype(np.int32)
    hist = [list(prompt[b]) for b in range(B)]
    nxt = sampled.prefill(prompt)
    plain.prefill(prompt)
    for step in range(20):
        logits = plain.logits()
        want = [oracle.sample_with_state(logits[b].copy(), hist[b], cfg, states[b]) for b in range(B)]
        assert nxt.tolist() == want, f"step {step}"
        for b in range(B):
            hist[b].append(int(nxt[b]))
        fed = nxt.copy()
        nxt = sampled.step_host(fed)
        plain.step_host(fed)
    # reset starts history and streams afresh: the same generation again
    sampled.reset()
    assert sampled.prefill(prompt).tolist() == [oracle.sample_with_state(
        _first_logits(plain, prompt)[b].copy(), list(prompt[b]), cfg, oracle.rng_state(33 + b)) for b in range(B)]
    sampled.set_sampling(None)
    sampled.reset()
    plain.reset()
    assert sampled.prefill(prompt).tolist() == plain.prefill(prompt).tolist()        # greedy again
    sampled.close()
    plain.close()


def _first_logits(plain, prompt):
    plain.reset()
    plain.prefill(prompt)
    return plain.logits()


def test_score_tokens(oracle):
    from test_model_oracle_vs_ref import oracle_score
    model = cached_model(oracle, TINY, seed=2)
    dec = CudaDecoder(model, batch=1, max_ctx=700)
    tokens = np.random.default_rng(9).integers(0, TINY["vocab"], 40).astype(np.int32)
    mask = np.ones(40, np.uint8)
    mask[5:12] = 0
    for m in (None, mask):
        dec.reset()
        got, n = dec.score_tokens(tokens, m)
        want, nw = oracle_score(oracle, OracleDecoder(oracle, model, max_ctx=64), tokens, m)
        assert n == nw
        assert abs(got - want) <= 2e-3 * abs(want), (got, want)
    # the state afterwards is the prompt's: decoding continues from it
    dec.reset()
    dec.score_tokens(tokens)
    a = dec.step_host([7])
    dec.reset()
    dec.prefill(tokens[None, :])
    assert dec.step_host([7]).tolist() == a.tolist()
    # longer than one lm_head group (512 rows) and the degenerate lengths
    dec.reset()
    long = np.random.default_rng(10).integers(0, TINY["vocab"], 650).astype(np.int32)
    nll, n = dec.score_tokens(long)
    assert n == 649 and 0.5 * np.log(TINY["vocab"]) < nll < 2.0 * np.log(TINY["vocab"])
    dec.reset()
    assert dec.score_tokens(long[:1]) == (0.0, 0)
    dec.close()
