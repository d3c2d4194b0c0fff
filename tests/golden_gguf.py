"""The tensors of the GGUF fixture tests/golden/tiny.gguf (written by the reference engine's
own GGUFWriter through oracle/_ref; tests/golden/make_golden.py gguf) - shared by the
generator and the tests, which regenerate the fp32 sources from the seeds here."""
import numpy as np

# GGML type ids (format/gguf_codec.h:35-50)
F32, F16, Q4_0, Q4_1, Q8_0 = 0, 1, 2, 3, 8
KIND_OF_GGML = {F32: -2, F16: -1, Q4_0: 0, Q4_1: 1, Q8_0: 2}

# (name, rows, cols (0 = one-dimensional), GGML type in the file)
TENSORS = [
    ("tok_embeddings", 32, 64, F16),
    ("layers.0.attn_norm", 64, 0, F32),
    ("layers.0.mamba.in_proj", 16, 64, Q4_0),
    ("layers.0.mamba.dt_bias", 32, 0, F32),
    ("layers.0.mamba.out_proj", 8, 64, Q8_0),
    ("layers.0.moe_router", 4, 64, F32),
    ("layers.0.moe_gate", 8, 64, Q4_1),
    ("layers.0.moe_up", 8, 64, Q4_0),
]


def source(name):
    """fp32 source of a fixture tensor (deterministic per name)."""
    i = [t[0] for t in TENSORS].index(name)
    _, rows, cols, _ = TENSORS[i]
    r = np.random.default_rng(1000 + i)
    n = rows * max(cols, 1)
    a = (r.standard_normal(n) * 0.05).astype(np.float32)
    if name.endswith("dt_bias"):
        a = r.uniform(-11.94, -0.58, n).astype(np.float32)        # mostly negative: the signed-extreme rule matters
    if name.endswith("moe_up"):
        a[:32] = 0.0                                               # a zero block
        a[32:64] = np.float32(-0.25)                               # every element the extreme: the first one wins
        a[64:96] = np.abs(a[64:96])                                # all positive
        a[100] = -a[96:128].max() - 1                              # a negative extreme among positives
    return a
