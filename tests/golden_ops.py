"""The golden-vector cases: for every op of the hot path one small seeded input set,
the call that runs it on a CPU backend (`Oracle` or `Ref`: same method names) and
the call that runs it through the CUDA C ABI.

tests/golden/make_golden.py runs `cpu()` of each case on the reference engine's own
compiled CPU objects and stores inputs and outputs in tests/golden/ops.npz;
tests/test_golden.py replays the stored inputs on the scalar oracle (no GPU) and on
the CUDA path (GPU) and compares with the stored outputs.  Inputs are stored, not
re-drawn, so the fixtures do not depend on the random generator of the test host.

Every case is a dict:
  name    unique key, prefix of its arrays in the .npz
  inputs  {str: ndarray}            (scalars as 0-d arrays)
  cpu     f(backend, inputs) -> {str: ndarray}
  gpu     f(inputs) -> {str: ndarray}   or None
  cpu_tol / gpu_tol   {output: "exact" | ("ulp", n) | (rtol, atol)}
"""
import numpy as np

EXACT = "exact"
SUM = (2e-4, 2e-5)          # fp32, differs by summation order only
ACT = (1e-2, 2e-2)          # stated activation bound vs the fp16-rounding CPU path


def _rng(seed):
    return np.random.default_rng(seed)


# ---------------------------------------------------------------------------
# block formats
# ---------------------------------------------------------------------------
def _quant_case(kind):
    x = (_rng(100 + kind).standard_normal(32 * 64) * 0.02).astype(np.float32)
    x[5] = 0.0
    x[64:96] = 0.0                       # all-zero block
    x[128:160] = np.abs(x[128:160])      # one-signed block
    x[200] = 3.0                         # outlier sets the scale of its block

    def cpu(b, inp):
        p = b.quantize(inp["x"], kind)
        return {"packed": p, "f16": b.dequantize(p, inp["x"].size, kind),
                "f32": b.dequantize_f32(p, inp["x"].size, kind)}

    def gpu(inp):
        import torch
        from gpu_util import dev, empty, host, ops, pkg
        from oracle_lib import packed_bytes
        n = inp["x"].size
        packed = empty(packed_bytes(kind, n), torch.uint8)
        pkg.lib().b200_quantize(dev(inp["x"]), packed, n, kind)
        back = empty(n, torch.int16)
        ops.dequantize_quant(packed, back, n, kind)
        return {"packed": host(packed), "f16": host(back, np.uint16)}

    return dict(name=f"quant_k{kind}", inputs={"x": x}, cpu=cpu, gpu=gpu,
                cpu_tol={"packed": EXACT, "f16": EXACT, "f32": EXACT},
                gpu_tol={"packed": EXACT, "f16": EXACT})


# ---------------------------------------------------------------------------
# linears
# ---------------------------------------------------------------------------
def _linear_case(oracle, wkind):
    M, K, N = 3, 96, 17
    r = _rng(110 + wkind)
    wf = (r.standard_normal((N, K)) * 0.05).astype(np.float32)
    if wkind == -2:
        w = wf
    elif wkind == -1:
        w = oracle.f32_to_f16(wf)
    else:
        w = oracle.quantize(wf.reshape(-1), wkind)
    x = r.standard_normal((M, K)).astype(np.float32)

    def cpu(b, inp):
        return {"y": b.linear(inp["x"], inp["w"], wkind, M, K, N)}

    def gpu(inp):
        from gpu_util import dev, empty, host, ops
        y = empty((M, N))
        if wkind == -2:
            ops.linear_forward_f32(dev(inp["x"]), dev(inp["w"]), y, M, K, N)
        elif wkind == -1:
            ops.linear_forward_fp16(dev(inp["x"]), dev(inp["w"]), y, M, K, N)
        else:
            ops.linear_forward_q4(dev(inp["x"]), dev(inp["w"]), y, M, K, N, wkind)
        return {"y": host(y)}

    return dict(name=f"linear_w{wkind}", inputs={"x": x, "w": w}, cpu=cpu, gpu=gpu,
                cpu_tol={"y": (1e-5, 1e-6) if wkind == -2 else EXACT},
                gpu_tol={"y": SUM if wkind < 0 else ACT})


# ---------------------------------------------------------------------------
# small ops
# ---------------------------------------------------------------------------
def _small_cases():
    r = _rng(130)
    cases = []

    x = r.standard_normal((5, 96)).astype(np.float32)
    x[3] = 0.0                                       # an all-zero row
    w = r.standard_normal(96).astype(np.float32)

    def rms_cpu(b, inp):
        out, rr = b.rmsnorm(inp["x"], inp["w"], 1e-5, True)
        return {"out": out, "rrms": rr}

    def rms_gpu(inp):
        from gpu_util import dev, empty, host, ops
        out, rr = empty((5, 96)), empty(5)
        ops.rmsnorm_forward(dev(inp["x"]), dev(inp["w"]), out, rr, 5, 96, 1e-5)
        return {"out": host(out), "rrms": host(rr)}

    cases.append(dict(name="rmsnorm", inputs={"x": x, "w": w}, cpu=rms_cpu, gpu=rms_gpu,
                      cpu_tol={"out": EXACT, "rrms": EXACT}, gpu_tol={"out": (1e-6, 1e-7), "rrms": (1e-6, 0)}))

    g = (r.standard_normal(300) * 3).astype(np.float32)
    u = r.standard_normal(300).astype(np.float32)
    g[0], g[1] = 50.0, -50.0

    def sw_cpu(b, inp):
        return {"out": b.swiglu(inp["g"], inp["u"])}

    def sw_gpu(inp):
        from gpu_util import dev, empty, host, ops
        out = empty(300)
        ops.swiglu_forward(dev(inp["g"]), dev(inp["u"]), out, 300)
        return {"out": host(out)}

    cases.append(dict(name="swiglu", inputs={"g": g, "u": u}, cpu=sw_cpu, gpu=sw_gpu,
                      cpu_tol={"out": EXACT}, gpu_tol={"out": (2e-6, 1e-7)}))

    tab = r.standard_normal((50, 16)).astype(np.float32)
    tabh = tab.astype(np.float16).view(np.uint16)
    ids = np.array([0, 49, -1, 50, 7], np.int32)     # out-of-range ids give zero rows

    def emb_cpu(b, inp):
        return {"f32": b.embedding(inp["ids"], inp["tab"], False, 16, 50),
                "f16": b.embedding(inp["ids"], inp["tabh"], True, 16, 50)}

    def emb_gpu(inp):
        from gpu_util import dev, empty, host, ops
        a, h = empty((5, 16)), empty((5, 16))
        ops.embedding_forward(dev(inp["ids"]), dev(inp["tab"]), a, 5, 16, 50)
        ops.embedding_forward_half(dev(inp["ids"]), dev(inp["tabh"]), h, 5, 16, 50)
        return {"f32": host(a), "f16": host(h)}

    cases.append(dict(name="embedding", inputs={"ids": ids, "tab": tab, "tabh": tabh}, cpu=emb_cpu, gpu=emb_gpu,
                      cpu_tol={"f32": EXACT, "f16": EXACT}, gpu_tol={"f32": EXACT, "f16": EXACT}))

    for rope_type in (0, 1):
        q = r.standard_normal((4, 6, 32)).astype(np.float32)
        k = r.standard_normal((4, 2, 32)).astype(np.float32)
        pos = np.array([0, 1, 77, 4095], np.int32)
        inv = (1.0 / 10000.0 ** (np.arange(16) / 16.0)).astype(np.float32)

        def rope_cpu(b, inp, rope_type=rope_type):
            qa, ka = b.rope_cached(inp["q"], inp["k"], inp["pos"], inp["inv"], 6, 2, 32, rope_type)
            return {"q": qa, "k": ka}

        def rope_gpu(inp, rope_type=rope_type):
            from gpu_util import dev, host, ops
            dq, dk = dev(inp["q"]), dev(inp["k"])
            ops.rope_forward_cached(dq, dk, dev(inp["pos"]), dev(inp["inv"]), 4, 6, 2, 32, rope_type)
            return {"q": host(dq), "k": host(dk)}

        cases.append(dict(name=f"rope_t{rope_type}", inputs={"q": q, "k": k, "pos": pos, "inv": inv},
                          cpu=rope_cpu, gpu=rope_gpu, cpu_tol={"q": EXACT, "k": EXACT},
                          gpu_tol={"q": (1e-4, 1e-4), "k": (1e-4, 1e-4)}))
    return cases


def _sampling_case():
    r = _rng(140)
    logits = r.standard_normal(1000).astype(np.float32)
    logits[10] = logits[500] = logits.max() + 1.0      # tie: the lowest id wins
    hist = np.array([10, 10, 999, -5, 2000, 7], np.int32)

    def cpu(b, inp):
        v, i = b.topk(inp["logits"], 8)
        return {"argmax": np.array([b.argmax(inp["logits"])], np.int32), "top_v": v, "top_i": i,
                "pen": b.rep_penalties(inp["logits"], inp["hist"], 1.12, 0.1, 0.2)}

    def gpu(inp):
        import ctypes as C
        import torch
        from gpu_util import dev, empty, host, ops
        dl = dev(inp["logits"])
        tok = C.c_int32(-1)
        ops.argmax_token(dl, 1000, C.byref(tok))
        v, i = empty(8), empty(8, torch.int32)
        ops.topk_select(dl, 1000, 8, v, i)
        pen = dev(inp["logits"])
        ops.apply_rep_penalties(pen, 1000, dev(inp["hist"]), 6, 1.12, 0.1, 0.2)
        return {"argmax": np.array([tok.value], np.int32), "top_v": host(v), "top_i": host(i), "pen": host(pen)}

    tol = {"argmax": EXACT, "top_v": EXACT, "top_i": EXACT, "pen": EXACT}
    return dict(name="sampling", inputs={"logits": logits, "hist": hist}, cpu=cpu, gpu=gpu, cpu_tol=tol,
                gpu_tol=dict(tol, pen=(1e-6, 1e-7)))


# ---------------------------------------------------------------------------
# MoE layer
# ---------------------------------------------------------------------------
def _moe_case(oracle, wkind, ne, K, SH, seed, d=64, E=32):
    from cases import moe_case
    N = 9
    c = moe_case(oracle, seed=seed, N=N, d=d, E=E, ne=ne, K=K, SH=SH, wkind=wkind,
                 bias_sigma=0.02 if SH else 0.0)
    keys = ("x", "router_w", "router_bias", "gates", "ups", "downs", "sh_g", "sh_u", "sh_d")
    inputs = {k: c[k] for k in keys if c[k] is not None}

    def cpu(b, inp):
        out, probs, idx, w = b.moe_forward(*[inp.get(k) for k in keys], d, E, ne, K, SH, wkind)
        return {"out": out, "probs": probs, "idx": idx, "w": w}

    def gpu(inp):
        import torch
        from gpu_util import dev, empty, host, ops
        out, probs, idx, w = empty((N, d)), empty((N, ne)), empty((N, K), torch.int32), empty((N, K))
        a = [dev(inp.get(k)) for k in keys]
        if wkind == -2:
            ops.moe_forward_bias(*a, out, probs, idx, w, None, None, None, N, d, E, ne, K, SH)
        else:
            ops.moe_forward_bias_half(*a, out, probs, idx, w, None, None, None, N, d, E, ne, K, SH, wkind)
        return {"out": host(out), "probs": host(probs), "idx": host(idx), "w": host(w)}

    return dict(name=f"moe_w{wkind}_e{ne}_k{K}", inputs=inputs, cpu=cpu, gpu=gpu,
                cpu_tol={"out": (2e-5, 2e-6), "probs": EXACT, "idx": EXACT, "w": EXACT},
                gpu_tol={"out": SUM if wkind < 0 else ACT, "probs": ("ulp", 4), "idx": EXACT, "w": ("ulp", 4)})


# ---------------------------------------------------------------------------
# Mamba-2 sequence forward
# ---------------------------------------------------------------------------
def _mamba_case(oracle, wkind):
    from cases import mamba_case
    c = mamba_case(oracle, seed=160, B=2, T=7, d=64, n_heads=4, d_head=32, d_state=16, k=4, wkind=wkind)
    names = ("x", "w_in", "conv_w", "conv_b", "dt_bias", "a_log", "D", "norm_w", "w_out", "state")
    inputs = dict(zip(names, c["args"][:10]))
    dims = c["args"][10:]                       # B, T, d, d_inner, conv_dim, n_heads, d_head, d_state, k, eps

    def cpu(b, inp):
        out, st = b.mamba2_forward(*[inp[n] for n in names], *dims, wkind)
        return {"out": out, "state": st}

    def gpu(inp):
        from gpu_util import dev, empty, host, ops
        a = [dev(inp[n]) for n in names]
        st = a[9].clone()
        out = empty((dims[0], dims[1], dims[2]))
        if wkind == -2:
            ops.mamba2_forward(*a[:9], st, out, *dims)
        else:
            ops.mamba2_forward_half(*a[:9], st, out, *dims, wkind)
        return {"out": host(out), "state": host(st)}

    return dict(name=f"mamba_w{wkind}", inputs=inputs, cpu=cpu, gpu=gpu,
                cpu_tol={"out": (2e-5, 2e-6), "state": (2e-5, 2e-7)},
                gpu_tol={"out": SUM if wkind < 0 else ACT, "state": SUM if wkind < 0 else ACT})


# ---------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------
def _attention_cases():
    r = _rng(170)
    B, T, H, KV, hd = 2, 9, 4, 2, 32
    q = r.standard_normal((B, T, H, hd)).astype(np.float32)
    k = r.standard_normal((B, T, KV, hd)).astype(np.float32)
    v = r.standard_normal((B, T, KV, hd)).astype(np.float32)
    seg = np.array([[0, 0, 0, 1, 1, 1, 1, 2, 2], [0] * 9], np.int32)
    cases = []
    for tag, window, use_seg in (("causal", 0, False), ("window3", 3, False), ("segments", 0, True)):
        inputs = {"q": q, "k": k, "v": v}
        if use_seg:
            inputs["seg"] = seg

        def cpu(b, inp, window=window):
            out, probs = b.attention_forward(inp["q"], inp["k"], inp["v"], B, T, H, KV, hd, 0.25, window,
                                             inp.get("seg"), True)
            return {"out": out, "probs": probs}

        def gpu(inp, window=window):
            from gpu_util import dev, empty, host, ops
            out, probs = empty((B, T, H, hd)), empty((B, H, T, T))
            ops.attention_forward_ex(dev(inp["q"]), dev(inp["k"]), dev(inp["v"]), out, probs, B, T, H, KV, hd,
                                     0.25, window, dev(inp.get("seg")))
            return {"out": host(out), "probs": host(probs)}

        cases.append(dict(name=f"attn_{tag}", inputs=inputs, cpu=cpu, gpu=gpu,
                          cpu_tol={"out": (1e-5, 1e-6), "probs": (1e-5, 1e-7)},
                          gpu_tol={"out": SUM, "probs": (2e-4, 1e-6)}))

    Hd, KVd, hdd, cache_max = 6, 2, 32, 24
    qd = r.standard_normal((Hd, hdd)).astype(np.float32)
    kc = r.standard_normal((cache_max, KVd * hdd)).astype(np.float32)
    vc = r.standard_normal((cache_max, KVd * hdd)).astype(np.float32)
    rings = ((0, 0, 1, 0), (0, 0, 24, 0), (5, 4, 24, 0), (0, 0, 17, 6), (3, 0, 20, 0))
    for half in (0, 1):
        kk, vv = (kc, vc) if not half else (kc.astype(np.float16).view(np.uint16),
                                            vc.astype(np.float16).view(np.uint16))

        def cpu(b, inp, half=half):
            return {f"o{n}": b.attention_decode_ring(inp["q"], inp["kc"], inp["vc"], half, Hd, KVd, hdd, rs, pin, cur,
                                                     cache_max, 0.2, win)
                    for n, (rs, pin, cur, win) in enumerate(rings)}

        def gpu(inp, half=half):
            from gpu_util import dev, empty, host, ops
            f = ops.attention_decode_ring_fp16 if half else ops.attention_decode_ring
            res = {}
            for n, (rs, pin, cur, win) in enumerate(rings):
                out = empty((Hd, hdd))
                f(dev(inp["q"]), dev(inp["kc"]), dev(inp["vc"]), out, Hd, KVd, hdd, rs, pin, cur, cache_max, 0.2,
                  None, win)
                res[f"o{n}"] = host(out)
            return res

        tol_c = {f"o{n}": (1e-5, 1e-6) for n in range(len(rings))}
        tol_g = {f"o{n}": SUM for n in range(len(rings))}
        cases.append(dict(name=f"attn_ring_h{half}", inputs={"q": qd, "kc": kk, "vc": vv}, cpu=cpu, gpu=gpu,
                          cpu_tol=tol_c, gpu_tol=tol_g))
    return cases


def all_cases(oracle):
    """`oracle` is only used to pack the seeded weights (its quantisers are pinned
    bit for bit to the reference's)."""
    cases = [_quant_case(k) for k in (0, 1, 2)]
    cases += [_linear_case(oracle, wk) for wk in (-2, -1, 0, 1, 2)]
    cases += _small_cases()
    cases.append(_sampling_case())
    cases += [_moe_case(oracle, -2, 8, 2, 64, 150), _moe_case(oracle, -1, 8, 2, 64, 151),
              _moe_case(oracle, 2, 8, 2, 64, 152), _moe_case(oracle, 0, 8, 2, 64, 153),
              _moe_case(oracle, -1, 64, 8, 0, 154, d=32, E=32)]
    cases += [_mamba_case(oracle, wk) for wk in (-2, -1, 2, 1)]
    cases += _attention_cases()
    return cases
