"""Golden vectors: outputs of the reference engine's own compiled CPU code, stored in
tests/golden/ by tests/golden/make_golden.py.  The scalar oracle must reproduce
them (no GPU needed), and so must the CUDA path through the C ABI (GPU), each
within the tolerance written beside the case in tests/golden_ops.py."""
import os

import numpy as np
import pytest

import golden_ops
from golden.make_golden import GOLDEN_MODEL, MODEL_ARRAYS
from oracle_lib import OracleOnly

HERE = os.path.dirname(os.path.abspath(__file__))
OPS = np.load(os.path.join(HERE, "golden", "ops.npz"))
MODEL = np.load(os.path.join(HERE, "golden", "model.npz"))
CASES = {c["name"]: c for c in golden_ops.all_cases(OracleOnly())}


def _stored(case, part):
    prefix = f"{case}/{part}/"
    return {k[len(prefix):]: OPS[k] for k in OPS.files if k.startswith(prefix)}


def _compare(got, want, tol, what):
    assert got.shape == want.shape, what
    if tol == golden_ops.EXACT:
        same = got.view(np.uint8) == want.view(np.uint8) if got.dtype == want.dtype else got == want
        assert np.all(same), f"{what}: {np.count_nonzero(~np.asarray(same))} bytes differ"
    elif tol[0] == "ulp":
        np.testing.assert_array_max_ulp(got, want, maxulp=tol[1])
    else:
        np.testing.assert_allclose(got, want, rtol=tol[0], atol=tol[1], err_msg=what)


def test_every_case_is_stored():
    stored = {k.split("/")[0] for k in OPS.files}
    assert stored == set(CASES), stored ^ set(CASES)


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_reproduces_reference_outputs(oracle, name):
    case = CASES[name]
    got = case["cpu"](oracle, _stored(name, "in"))
    want = _stored(name, "out")
    assert set(got) == set(want)
    for k in want:
        _compare(np.asarray(got[k]), want[k], case["cpu_tol"][k], f"{name}/{k}")


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(CASES))
def test_cuda_reproduces_reference_outputs(name):
    case = CASES[name]
    got = case["gpu"](_stored(name, "in"))
    want = _stored(name, "out")
    for k, v in got.items():
        _compare(np.asarray(v), want[k], case["gpu_tol"][k], f"{name}/{k}")


def _golden_model():
    cfg = GOLDEN_MODEL
    d_inner = cfg["mamba_heads"] * cfg["mamba_d_head"]
    m = {"cfg": cfg, "layers": []}
    for k in MODEL_ARRAYS:
        m[k] = MODEL[k]
    for i, t in enumerate(cfg["layer_types"]):
        prefix = f"layer{i}/"
        L = {k[len(prefix):]: MODEL[k] for k in MODEL.files if k.startswith(prefix)}
        L.update(type=t, router_bias=None, d_inner=d_inner, conv_dim=d_inner + 2 * cfg["mamba_d_state"])
        m["layers"].append(L)
    return m


def test_oracle_decoder_reproduces_reference_generator(oracle):
    """Model level: the per-token walk over the oracle against the logits of the
    reference's Model + Generator; greedy picks identical."""
    from model_util import OracleDecoder
    dec = OracleDecoder(oracle, _golden_model(), max_ctx=16)
    for tok, want in zip(MODEL["tokens"], MODEL["logits"]):
        got = dec.step(int(tok))
        np.testing.assert_allclose(got, want, rtol=2e-4, atol=2e-5)
        assert int(np.argmax(got)) == int(np.argmax(want))


@pytest.mark.gpu
@pytest.mark.parametrize("fused,graph", [(0, 0), (1, 1)])
def test_cuda_decoder_reproduces_reference_generator(fused, graph):
    """The CUDA decoder against the reference CPU logits: the stated activation bound
    (rel 1e-2 / abs 2e-2) and the same greedy token wherever the reference's top-2
    margin exceeds that bound."""
    from gpu_util import ACTIVATION
    from model_util import CudaDecoder
    dec = CudaDecoder(_golden_model(), batch=1, max_ctx=16, kv_page=16)
    dec.configure(fused, graph)
    for tok, want in zip(MODEL["tokens"], MODEL["logits"]):
        nxt = dec.step_host([int(tok)])
        got = dec.logits()[0]
        np.testing.assert_allclose(got, want, **ACTIVATION)
        top2 = np.sort(want)[-2:]
        if top2[1] - top2[0] > 4e-2:
            assert int(nxt[0]) == int(np.argmax(want))
    dec.close()
