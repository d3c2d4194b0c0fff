"""GPU parity of the prompt path: b200_decoder_prefill (many-token kernels: tensor-core
GEMMs, chunked SSD scan, tensor-core attention, grouped MoE) against the same prompt fed
one token at a time, and against the oracle's per-token walk."""
import numpy as np
import pytest

from gpu_util import fp16_close
from model_util import CONFIG_1, TINY, CudaDecoder, OracleDecoder, make_model

pytestmark = pytest.mark.gpu


def _stepwise(dec, prompt):
    nxt = None
    for t in range(prompt.shape[1]):
        nxt = dec.step_host(prompt[:, t])
    return nxt, dec.logits()


@pytest.mark.parametrize("T", [1, 5, 48, 200])
def test_prefill_matches_stepwise_decode(oracle, T):
    """Short prompts take the per-row kernels (fp32), long ones the tensor-core path
    (fp16 operands): logits agree within the fp16 scale-relative bound either way, and
    the state handed over (ssm state, conv window, KV pages, lengths) continues the
    sequence exactly like the stepwise decoder's."""
    B = 2
    model = make_model(oracle, TINY, 5)
    r = np.random.default_rng(T)
    prompt = r.integers(0, TINY["vocab"], (B, T))
    a = CudaDecoder(model, batch=B, max_ctx=T + 8)
    b = CudaDecoder(model, batch=B, max_ctx=T + 8)
    _, want = _stepwise(a, prompt)
    got_next = b.prefill(prompt)
    got = b.logits()
    fp16_close(got, want)
    assert np.array_equal(got_next, got.argmax(axis=1))
    # continue both for a few tokens on the same inputs
    for s in range(4):
        toks = r.integers(0, TINY["vocab"], B)
        a.step_host(toks)
        b.step_host(toks)
        fp16_close(b.logits(), a.logits())
    a.close()
    b.close()


def test_prefill_matches_oracle(oracle):
    cfg = dict(CONFIG_1, vocab=2048)
    T = 40
    model = make_model(oracle, cfg, 9)
    prompt = np.random.default_rng(2).integers(0, cfg["vocab"], (1, T))
    ora = OracleDecoder(oracle, model, max_ctx=T + 4)
    want = None
    for t in range(T):
        want = ora.step(int(prompt[0, t]))
    dec = CudaDecoder(model, batch=1, max_ctx=T + 4)
    nxt = dec.prefill(prompt)
    got = dec.logits()[0]
    err = np.abs(got - want)
    assert np.all(err <= 2e-2 + 1e-2 * np.abs(want)), f"max abs err {err.max()}"
    top2 = np.sort(want)[-2:]
    if top2[1] - top2[0] > 1e-3:
        assert int(nxt[0]) == oracle.argmax(want)
    # the next decoded token continues from the prefilled state
    tok = int(nxt[0])
    want2 = ora.step(tok)
    dec.step_host([tok])
    err = np.abs(dec.logits()[0] - want2)
    assert np.all(err <= 2e-2 + 1e-2 * np.abs(want2)), f"max abs err {err.max()}"
    dec.close()


def test_prefill_4096_tokens_at_h_tiny_widths(oracle):
    """A 4096-token prompt through the four-layer cut at the H-Tiny widths (Mamba, attention,
    Mamba, Mamba, an MoE after each; Q4_K): the prompt path against the same tokens fed
    through the decode step (which the oracle pins at these widths in
    tests/test_gpu_decoder.py), logits and the following steps; and the first 48 tokens of
    the same prompt against the oracle's own walk."""
    from model_util import cached_model
    from test_gpu_decoder import H_TINY_CUT
    cfg = H_TINY_CUT
    T = 4096
    model = cached_model(oracle, cfg, 0, share_experts=True)
    r = np.random.default_rng(22)
    prompt = r.integers(0, cfg["vocab"], (1, T))
    a = CudaDecoder(model, batch=1, max_ctx=T + 8)
    b = CudaDecoder(model, batch=1, max_ctx=T + 8)
    a.configure(1, 1)
    _, want = _stepwise(a, prompt)
    b.prefill(prompt)
    fp16_close(b.logits(), want)
    b.configure(2, 1)
    for s in range(4):
        toks = r.integers(0, cfg["vocab"], 1)
        a.step_host(toks)
        b.step_host(toks)
        fp16_close(b.logits(), a.logits())
    a.close()
    b.close()
    # oracle: 48 tokens of the same prompt
    T0 = 48
    ora = OracleDecoder(oracle, model, max_ctx=T0 + 4)
    for t in range(T0):
        want0 = ora.step(int(prompt[0, t]))
    c = CudaDecoder(model, batch=1, max_ctx=T0 + 8)
    c.prefill(prompt[:, :T0])
    err = np.abs(c.logits()[0] - want0)
    assert np.all(err <= 2e-2 + 1e-2 * np.abs(want0)), f"max abs err {err.max()}"
    c.close()


def test_prefill_needs_empty_sequences(oracle):
    model = make_model(oracle, TINY, 1)
    dec = CudaDecoder(model, batch=1, max_ctx=16)
    dec.step_host([3])
    with pytest.raises(Exception):
        dec.prefill(np.zeros((1, 4), np.int32))
    dec.reset()
    with pytest.raises(Exception):
        dec.prefill(np.zeros((1, 65), np.int32))      # longer than the context (16 rounds up to one 64-token page)
    dec.prefill(np.zeros((1, 4), np.int32))
    with pytest.raises(Exception):
        dec.prefill(np.zeros((1, 4), np.int32))       # sequences no longer empty
    dec.close()


def test_prefill_fp16_weights_and_reset(oracle):
    """qkind -1 (fp16 matrices: the GEMM without the in-kernel expansion), and a second prompt
    after reset reproduces the first run bit for bit (no state leaks through the workspaces)."""
    cfg = dict(TINY, qkind=-1)
    model = make_model(oracle, cfg, 11)
    prompt = np.random.default_rng(3).integers(0, cfg["vocab"], (2, 150))
    a = CudaDecoder(model, batch=2, max_ctx=160)
    b = CudaDecoder(model, batch=2, max_ctx=160)
    _, want = _stepwise(a, prompt)
    b.prefill(prompt)
    first = b.logits().copy()
    fp16_close(first, want)
    b.reset()
    b.prefill(prompt)
    assert np.array_equal(b.logits(), first)
    a.close()
    b.close()


RAGGED = [1, 63, 64, 129, 300, 2, 128, 257]


@pytest.mark.parametrize("cfg_name", ["tiny", "narrow_heads"])
def test_ragged_prefill_matches_one_sequence_at_a_time(oracle, cfg_name):
    """Prompts of different lengths in one batch (b200_decoder_prefill_ragged): every sequence
    ends where its own single-sequence prefill ends (logits, pick), and the batch then decodes
    on, each sequence at its own position, like the single decoders do.  'narrow_heads' has a
    Mamba head width outside the chunked scan's tiling, so its scan runs per sequence."""
    cfg = TINY if cfg_name == "tiny" else dict(TINY, mamba_heads=16, mamba_d_head=32, mamba_d_state=64)
    model = make_model(oracle, cfg, 6)
    r = np.random.default_rng(11)
    prompts = [r.integers(0, cfg["vocab"], n).astype(np.int32) for n in RAGGED]
    B = len(prompts)
    batch = CudaDecoder(model, batch=B, max_ctx=320)
    got_next = batch.prefill_ragged(prompts)
    got = batch.logits()
    singles = []
    for b, p in enumerate(prompts):
        one = CudaDecoder(model, batch=1, max_ctx=320)
        nxt = one.prefill(p[None, :])
        want = one.logits()[0]
        fp16_close(got[b], want)
        if np.sort(want)[-1] - np.sort(want)[-2] > 1e-2:          # a clear winner: the picks agree
            assert int(got_next[b]) == int(nxt[0])
        singles.append(one)
    assert np.array_equal(got_next, got.argmax(axis=1))
    for s in range(3):
        toks = r.integers(0, cfg["vocab"], B).astype(np.int32)
        batch.step_host(toks)
        now = batch.logits()
        for b, one in enumerate(singles):
            one.step_host(toks[b:b + 1])
            fp16_close(now[b], one.logits()[0])
    for one in singles:
        one.close()
    batch.close()


def test_ragged_prefill_rejects_bad_lengths(oracle):
    from gpu_util import B200Error
    model = make_model(oracle, TINY, 6)
    dec = CudaDecoder(model, batch=2, max_ctx=64)          # one KV page of 64 tokens
    with pytest.raises(B200Error):
        dec.prefill_ragged([np.zeros(0, np.int32), np.zeros(4, np.int32)])
    with pytest.raises(B200Error):
        dec.prefill_ragged([np.zeros(4, np.int32), np.zeros(65, np.int32)])
    assert dec.prefill_ragged([np.zeros(4, np.int32), np.ones(64, np.int32)]).shape == (2,)
    with pytest.raises(B200Error):                                     # not empty any more
        dec.prefill_ragged([np.zeros(4, np.int32), np.ones(4, np.int32)])
    dec.close()


def test_ragged_prefill_in_several_groups(oracle):
    """More tokens than one group holds (32768): the sequences are processed in groups of
    consecutive sequences; equal lengths must reproduce the rectangular prefill bit for bit
    where the grouping coincides."""
    cfg = dict(TINY, n_layers=2, layer_types=[0, 1])
    model = make_model(oracle, cfg, 7)
    r = np.random.default_rng(3)
    lengths = [9000, 12000, 20000, 700]
    prompts = [r.integers(0, cfg["vocab"], n).astype(np.int32) for n in lengths]
    dec = CudaDecoder(model, batch=4, max_ctx=20000)
    nxt = dec.prefill_ragged(prompts)
    got = dec.logits()
    one = CudaDecoder(model, batch=1, max_ctx=20000)
    for b in (2, 3):
        one.reset()
        one.prefill(prompts[b][None, :])
        fp16_close(got[b], one.logits()[0])
    assert np.array_equal(nxt, got.argmax(axis=1))
    one.close()
    dec.close()
