"""Generates the golden fixtures of this directory from the reference engine's own
compiled CPU code (oracle/_ref/libgai_ref.so, built by `make -C oracle` where the
reference sources are mounted).  Run from the repository root:

    python tests/golden/make_golden.py

ops.npz    per case of tests/golden_ops.py: "<case>/in/<name>" (the inputs) and
           "<case>/out/<name>" (what the reference's CPU objects returned).
model.npz  a two-layer hybrid model (Mamba-2 layer + GQA layer, MoE after each) in
           its stored form (Q8_0 matrices, fp16 embeddings), a token sequence, and the
           logits the reference's Model + Generator produced for each token on its
           CPU device from the same fp32 source weights.

config1.npz  (`python tests/golden/make_golden.py config1`, about twenty minutes of CPU)
           the 8-layer Q8_0 hybrid model of CONFIG_1 at its full vocabulary of 32768,
           weights from random_f32_params(CONFIG_1, seed 0): a 128-token prompt (uniform
           ids, seed 1) followed by 128 greedy steps of the reference's Model + Generator
           on its CPU device.  Stored per step: the token fed, the arg-max, the ids and
           values of the eight largest logits, and mean / max |logit| (the weights are
           regenerated from the seed at test time, so the file stays a few KB).

tiny.gguf  (`python tests/golden/make_golden.py gguf`) a GGUF v3 file written by the
           reference's own GGUFWriter (format/gguf_codec.cpp:514-640) from the tensors of
           tests/golden_gguf.py: F32, F16, Q8_0, Q4_1 and Q4_0 payloads (the last by the
           writer's signed-extreme rule, :408-460); gguf_expected.npz holds what the
           reference's GGUFReader returns for them (read_tensor_f32, and read_tensor_quant
           to Q8_0 / Q4_0 / Q4_1: the verbatim and the quantise-on-load paths).

sampler.npz (`python tests/golden/make_golden.py sampler`) draws of the reference's Sampler
           (inference/sampler.cpp) for the configurations of tests/sampler_cases.py, 500
           outputs of its generator (core/rng.h) and one cross-entropy sum (core/math_cpu.cpp:560).

The fixtures are read by tests/test_sampler_oracle.py, tests/test_golden.py, tests/test_gpu_golden_model.py and
tests/test_gguf.py; nothing at test time needs the reference sources.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

from golden_ops import all_cases                                     # noqa: E402
from model_util import RefGenerator, model_from_f32, random_f32_params   # noqa: E402
from oracle_lib import OracleOnly, Ref                               # noqa: E402

GOLDEN_MODEL = dict(vocab=96, hidden=64, n_layers=2, layer_types=[0, 1],
                    n_heads=2, n_kv=1, head_dim=32, rope_type=1, rope_theta=1e4,
                    mamba_heads=4, mamba_d_head=16, mamba_d_state=32, mamba_d_conv=4,
                    n_experts=4, top_k=2, expert_dim=32, shared_dim=32, qkind=2,
                    rms_eps=1e-5, embedding_multiplier=12.0, residual_multiplier=0.22,
                    attn_scale=0.0078125, logits_scaling=6.0)
GOLDEN_TOKENS = [5, 17, 0, 95, 42, 42, 7, 63, 1, 30]
MODEL_ARRAYS = ("embed", "final_norm", "inv_freq")


def make_ops(oracle, ref):
    out = {}
    for case in all_cases(oracle):
        for k, v in case["inputs"].items():
            out[f"{case['name']}/in/{k}"] = np.asarray(v)
        for k, v in case["cpu"](ref, case["inputs"]).items():
            out[f"{case['name']}/out/{k}"] = np.asarray(v)
    return out


def make_model(oracle):
    cfg = GOLDEN_MODEL
    params = random_f32_params(cfg, seed=11)
    gen = RefGenerator(cfg, params, max_ctx=16)
    logits = np.stack([gen.step(t) for t in GOLDEN_TOKENS])
    gen.close()
    m = model_from_f32(oracle, cfg, params)
    out = {"tokens": np.array(GOLDEN_TOKENS, np.int32), "logits": logits}
    for k in MODEL_ARRAYS:
        out[k] = m[k]
    for i, L in enumerate(m["layers"]):
        for k, v in L.items():
            if isinstance(v, np.ndarray):
                out[f"layer{i}/{k}"] = v
    return out


CONFIG1_PROMPT, CONFIG1_STEPS, CONFIG1_TOP = 128, 128, 8


def make_config1():
    from model_util import CONFIG_1
    cfg = CONFIG_1
    params = random_f32_params(cfg, seed=0)
    total = CONFIG1_PROMPT + CONFIG1_STEPS
    gen = RefGenerator(cfg, params, max_ctx=total + 1)
    prompt = np.random.default_rng(1).integers(0, cfg["vocab"], CONFIG1_PROMPT)
    fed = np.zeros(total, np.int32)
    arg = np.zeros(total, np.int32)
    top_i = np.zeros((total, CONFIG1_TOP), np.int32)
    top_v = np.zeros((total, CONFIG1_TOP), np.float32)
    stats = np.zeros((total, 2), np.float32)
    tok = int(prompt[0])
    for s in range(total):
        logits = gen.step(tok)
        fed[s] = tok
        order = np.argsort(-logits, kind="stable")[:CONFIG1_TOP]
        top_i[s], top_v[s] = order, logits[order]
        arg[s] = order[0]
        stats[s] = (np.abs(logits).mean(), np.abs(logits).max())
        tok = int(prompt[s + 1]) if s + 1 < CONFIG1_PROMPT else int(arg[s])
        if s % 16 == 0:
            print("config1 step", s, flush=True)
    gen.close()
    return dict(fed=fed, argmax=arg, top_ids=top_i, top_vals=top_v, stats=stats,
                prompt_len=np.int32(CONFIG1_PROMPT))


def make_gguf():
    import ctypes as C
    import golden_gguf as gg
    from oracle_lib import ROOT
    lib = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libgai_ref.so"))
    lib.ref_last_error.restype = C.c_char_p
    path = os.path.join(HERE, "tiny.gguf")
    n = len(gg.TENSORS)
    srcs = [np.ascontiguousarray(gg.source(t[0])) for t in gg.TENSORS]
    names = (C.c_char_p * n)(*[t[0].encode() for t in gg.TENSORS])
    rows = (C.c_int64 * n)(*[t[1] for t in gg.TENSORS])
    cols = (C.c_int64 * n)(*[t[2] for t in gg.TENSORS])
    data = (C.c_void_p * n)(*[a.ctypes.data for a in srcs])
    types = (C.c_int * n)(*[t[3] for t in gg.TENSORS])
    if lib.ref_gguf_write(path.encode(), n, names, rows, cols, data, types) != 0:
        raise RuntimeError(lib.ref_last_error().decode())
    expected = {}
    for (name, r_, c_, _), a in zip(gg.TENSORS, srcs):
        for kind, label in ((-2, "f32"), (2, "q8_0"), (0, "q4_0"), (1, "q4_1")):
            if kind >= 0 and a.size % 32:
                continue
            buf = np.zeros(a.size * 4 + 64, np.uint8)
            nb = C.c_int64()
            if lib.ref_gguf_read(path.encode(), name.encode(), kind, buf.ctypes.data_as(C.c_void_p), C.c_int64(buf.size),
                                 C.byref(nb)) != 0:
                raise RuntimeError(lib.ref_last_error().decode())
            expected[f"{name}/{label}"] = buf[:nb.value].copy()
    np.savez_compressed(os.path.join(HERE, "gguf_expected.npz"), **expected)
    print("tiny.gguf", os.path.getsize(path), "bytes;", len(expected), "expected reads")


def make_sampler():
    import sampler_cases as sc
    from oracle_lib import Ref
    ref = Ref()
    out = {}
    for name, cfg in sc.CONFIGS.items():
        for seed in (1, 2):
            out[f"{name}/{seed}"] = ref.sample(sc.logits(seed), sc.history(seed), cfg, 77 + seed, sc.DRAWS)
    out["uniform/42"] = ref.rng_uniform(42, 500)
    t = np.array([5, -100, 999, 0], np.int32)
    total, count = ref.cross_entropy(sc.logits(3, 4000).reshape(4, 1000), t, 1e-4)
    out["ce/targets"], out["ce/sum"], out["ce/count"] = t, np.float64(total), np.int64(count)
    np.savez_compressed(os.path.join(HERE, "sampler.npz"), **out)
    print("sampler.npz:", len(out), "arrays")


def main():
    if len(sys.argv) > 1 and sys.argv[1] == "sampler":
        make_sampler()
        return
    if len(sys.argv) > 1 and sys.argv[1] == "gguf":
        make_gguf()
        return
    if len(sys.argv) > 1 and sys.argv[1] == "config1":
        np.savez_compressed(os.path.join(HERE, "config1.npz"), **make_config1())
        print("config1.npz", os.path.getsize(os.path.join(HERE, "config1.npz")), "bytes")
        return
    oracle, ref = OracleOnly(), Ref()
    np.savez_compressed(os.path.join(HERE, "ops.npz"), **make_ops(oracle, ref))
    np.savez_compressed(os.path.join(HERE, "model.npz"), **make_model(oracle))
    for f in ("ops.npz", "model.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
