"""Random-init hybrid models (Mamba-2 + GQA + MoE) for the model-level tests, the
Python restatement of the reference's per-token op sequence over the CPU oracle,
and the loader that hands the same bytes to the CUDA decoder.

Weight storage follows Model::storage_dtype_for (model/model.cpp:959-986): norms,
conv, dt_bias, A_log, D, router and router bias fp32; embeddings / lm_head fp16
(tied); every other matrix packed in the model's qkind.
"""
import ctypes as C

import numpy as np

from cases import mamba_params, store_weight

# config 1 of the benchmark description, scaled to a test-sized vocabulary
CONFIG_1 = dict(vocab=32768, hidden=768, n_layers=8, layer_types=[0, 0, 0, 1, 0, 0, 0, 1],
                n_heads=12, n_kv=4, head_dim=64, rope_type=1, rope_theta=1e4,
                mamba_heads=24, mamba_d_head=64, mamba_d_state=64, mamba_d_conv=4,
                n_experts=16, top_k=2, expert_dim=512, shared_dim=1024, qkind=2,
                rms_eps=1e-5, embedding_multiplier=1.0, residual_multiplier=1.0,
                attn_scale=0.0, logits_scaling=1.0)

TINY = dict(vocab=512, hidden=256, n_layers=4, layer_types=[0, 1, 0, 1],
            n_heads=4, n_kv=2, head_dim=64, rope_type=1, rope_theta=1e4,
            mamba_heads=8, mamba_d_head=64, mamba_d_state=128, mamba_d_conv=4,
            n_experts=8, top_k=2, expert_dim=256, shared_dim=256, qkind=3,
            rms_eps=1e-5, embedding_multiplier=12.0, residual_multiplier=0.22,
            attn_scale=0.0078125, logits_scaling=6.0)


class B200Sampling(C.Structure):
    """struct b200_sampling of include/b200step.h."""
    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("min_p", C.c_float), ("repetition_penalty", C.c_float),
                ("frequency_penalty", C.c_float), ("presence_penalty", C.c_float), ("top_k", C.c_int32),
                ("repetition_window", C.c_int32), ("no_repeat_ngram", C.c_int32), ("greedy", C.c_int32),
                ("seed", C.c_uint64)]

    @classmethod
    def of(cls, cfg, seed=0):
        """From an oracle_lib.Sampling."""
        return cls(cfg.temperature, cfg.top_p, cfg.min_p, cfg.repetition_penalty, cfg.frequency_penalty,
                   cfg.presence_penalty, cfg.top_k, cfg.repetition_window, cfg.no_repeat_ngram, int(cfg.greedy), seed)


_MODEL_CACHE = {}


def cached_model(oracle, cfg, seed=0, share_experts=False):
    """make_model() memoised per (configuration, seed): the wide test models take tens of
    seconds to draw and quantise."""
    key = (tuple(sorted((k, tuple(v) if isinstance(v, list) else v) for k, v in cfg.items())), seed, share_experts)
    if key not in _MODEL_CACHE:
        _MODEL_CACHE[key] = make_model(oracle, cfg, seed, share_experts=share_experts)
    return _MODEL_CACHE[key]


def make_model(oracle, cfg, seed=0, w_std=0.02, share_experts=False):
    """share_experts: every layer uses the same routed-expert matrices (drawn once; the wide
    models spend most of their set-up time there), everything else differs per layer."""
    r = np.random.default_rng(seed)
    shared = {}
    d, q = cfg["hidden"], cfg["qkind"]
    m = {"cfg": cfg, "layers": []}
    emb = (r.standard_normal((cfg["vocab"], d)) * w_std).astype(np.float32)
    m["embed"] = oracle.f32_to_f16(emb)                      # tied with lm_head
    m["final_norm"] = (1 + 0.1 * r.standard_normal(d)).astype(np.float32)
    hd = cfg["head_dim"]
    m["inv_freq"] = (1.0 / cfg["rope_theta"] ** (np.arange(hd // 2) * 2.0 / hd)).astype(np.float32)
    qd, kvd = cfg["n_heads"] * hd, cfg["n_kv"] * hd
    ne, E, SH = cfg["n_experts"], cfg["expert_dim"], cfg["shared_dim"]
    for t in cfg["layer_types"]:
        L = {"type": t,
             "attn_norm": (1 + 0.1 * r.standard_normal(d)).astype(np.float32),
             "ffn_norm": (1 + 0.1 * r.standard_normal(d)).astype(np.float32)}
        if t == 0:
            L.update(mamba_params(oracle, r, d, cfg["mamba_heads"], cfg["mamba_d_head"], cfg["mamba_d_state"],
                                  cfg["mamba_d_conv"], q, w_std))
        else:
            L["wq"] = store_weight(oracle, r.standard_normal((qd, d)) * w_std, q)
            L["wk"] = store_weight(oracle, r.standard_normal((kvd, d)) * w_std, q)
            L["wv"] = store_weight(oracle, r.standard_normal((kvd, d)) * w_std, q)
            L["wo"] = store_weight(oracle, r.standard_normal((d, qd)) * w_std, q)
        L["router"] = (r.standard_normal((ne, d)) / np.sqrt(d)).astype(np.float32)
        L["router_bias"] = (r.standard_normal(ne) * 0.5 / ne).astype(np.float32)
        if not (share_experts and shared):
            shared = dict(gate=store_weight(oracle, r.standard_normal((ne * E, d)) * w_std, q),
                          up=store_weight(oracle, r.standard_normal((ne * E, d)) * w_std, q),
                          down=store_weight(oracle, r.standard_normal((ne * d, E)) * w_std, q))
        L.update(shared if share_experts else dict(shared))
        if not share_experts:
            shared = {}
        L["sh_gate"] = store_weight(oracle, r.standard_normal((SH, d)) * w_std, q)
        L["sh_up"] = store_weight(oracle, r.standard_normal((SH, d)) * w_std, q)
        L["sh_down"] = store_weight(oracle, r.standard_normal((d, SH)) * w_std, q)
        m["layers"].append(L)
    return m


class OracleDecoder:
    """One sequence, one token at a time, in the op order of
    Generator::decode_step_logits (inference/generator.cpp:221-443) with the CPU
    oracle standing in for every op.  The KV cache is the reference's fp16 ring with
    no pinned prefix and ring_start 0 (a contiguous cache)."""

    def __init__(self, oracle, model, max_ctx, rope_as_reference=False):
        """rope_as_reference: mirror Generator::decode_step_logits' handling of the position
        word (inference/generator.cpp:340-345: uploaded only when layer 0 is an attention
        layer; otherwise every token is rotated by one stale angle, i.e. q.k is as without
        rotation)."""
        self.o, self.m, self.cfg = oracle, model, model["cfg"]
        self.rope = model["cfg"]["rope_type"] >= 0 and not (rope_as_reference and model["cfg"]["layer_types"][0] == 0)
        c = self.cfg
        self.max_ctx = max_ctx
        self.conv_dim = c["mamba_heads"] * c["mamba_d_head"] + 2 * c["mamba_d_state"]
        self.reset()

    def reset(self):
        c = self.cfg
        kvd = c["n_kv"] * c["head_dim"]
        self.pos = 0
        self.state = []
        for t in c["layer_types"]:
            if t == 0:
                self.state.append(dict(
                    conv=np.zeros((self.conv_dim, c["mamba_d_conv"] - 1), np.float32),
                    ssm=np.zeros((c["mamba_heads"] * c["mamba_d_head"], c["mamba_d_state"]), np.float32)))
            else:
                self.state.append(dict(k=np.zeros((self.max_ctx, kvd), np.uint16),
                                       v=np.zeros((self.max_ctx, kvd), np.uint16)))

    def step(self, token):
        o, c, m = self.o, self.cfg, self.m
        d, q = c["hidden"], c["qkind"]
        hd, H, KV = c["head_dim"], c["n_heads"], c["n_kv"]
        scale = c["attn_scale"] if c["attn_scale"] > 0 else 1.0 / np.sqrt(np.float32(hd))
        x = o.embedding(np.array([token], np.int32), m["embed"], True, d, c["vocab"])[0]
        if c["embedding_multiplier"] != 1.0:
            x = x * np.float32(c["embedding_multiplier"])
        for L, st in zip(m["layers"], self.state):
            xb = o.rmsnorm(x[None], L["attn_norm"], c["rms_eps"])[0]
            if L["type"] == 0:
                y, st["conv"], st["ssm"] = o.mamba2_step(
                    xb, L["w_in"], L["conv_w"], L["conv_b"], L["dt_bias"], L["a_log"], L["D"], L["norm_w"],
                    L["w_out"], st["conv"], st["ssm"], d, L["d_inner"], L["conv_dim"], c["mamba_heads"],
                    c["mamba_d_head"], c["mamba_d_state"], c["mamba_d_conv"], c["rms_eps"], q)
            else:
                qv = o.linear(xb[None], L["wq"], q, 1, d, H * hd)
                kv = o.linear(xb[None], L["wk"], q, 1, d, KV * hd)
                vv = o.linear(xb[None], L["wv"], q, 1, d, KV * hd)
                if self.rope:
                    qv, kv = o.rope_cached(qv.reshape(1, H, hd), kv.reshape(1, KV, hd),
                                           np.array([self.pos], np.int32), m["inv_freq"], H, KV, hd, c["rope_type"])
                st["k"][self.pos] = o.f32_to_f16(kv.reshape(-1))
                st["v"][self.pos] = o.f32_to_f16(vv.reshape(-1))
                a = o.attention_decode_ring(qv.reshape(H, hd), st["k"], st["v"], 1, H, KV, hd, 0, 0, self.pos + 1,
                                            self.max_ctx, float(scale), 0)
                y = o.linear(a.reshape(1, -1), L["wo"], q, 1, H * hd, d)[0]
            x = x + y * np.float32(c["residual_multiplier"])
            xb = o.rmsnorm(x[None], L["ffn_norm"], c["rms_eps"])
            y, _, _, _ = o.moe_forward(xb, L["router"], L["router_bias"], L["gate"], L["up"], L["down"], L["sh_gate"],
                                       L["sh_up"], L["sh_down"], d, c["expert_dim"], c["n_experts"], c["top_k"],
                                       c["shared_dim"], q)
            x = x + y[0] * np.float32(c["residual_multiplier"])
        xb = o.rmsnorm(x[None], m["final_norm"], c["rms_eps"])
        logits = o.linear(xb, m["embed"], -1, 1, d, c["vocab"])[0]
        if c["logits_scaling"] != 1.0:
            logits = logits * np.float32(1.0 / np.float32(c["logits_scaling"]))
        self.pos += 1
        return logits


# tensor ids of include/b200step.h
T = dict(embed=0, final_norm=1, lm_head=2, inv_freq=3, attn_norm=10, ffn_norm=11,
         w_in=20, conv_w=21, conv_b=22, dt_bias=23, a_log=24, D=25, norm_w=26, w_out=27,
         wq=30, wk=31, wv=32, wo=33, router=40, router_bias=41, gate=42, up=43, down=44,
         sh_gate=45, sh_up=46, sh_down=47)


class CudaDecoder:
    """b200_decoder over device copies of a make_model() model."""

    def __init__(self, model, batch, max_ctx, kv_page=64, rope_as_reference=False):
        from gpu_util import dev, pkg
        self.lib = pkg.lib()
        c = model["cfg"]
        self.cfg, self.batch = c, batch
        self.handle = C.c_void_p()
        types = np.array(c["layer_types"], np.int32)
        self.lib.b200_decoder_create(C.byref(self.handle), batch, c["vocab"], c["hidden"], c["n_layers"],
                                     types.ctypes.data, c["n_heads"], c["n_kv"], c["head_dim"], c["rope_type"],
                                     c["mamba_heads"], c["mamba_d_head"], c["mamba_d_state"], c["mamba_d_conv"],
                                     c["n_experts"], c["top_k"], c["expert_dim"], c["shared_dim"], max_ctx, kv_page,
                                     c["qkind"], c["rms_eps"], c["embedding_multiplier"], c["residual_multiplier"],
                                     c["attn_scale"], c["logits_scaling"])
        self.keep = []
        if rope_as_reference:
            self.lib.b200_decoder_set_rope_refresh(self.handle, 1)

        def put(layer, name, arr):
            t = dev(arr)
            self.keep.append(t)
            self.lib.b200_decoder_set_tensor(self.handle, layer, T[name], t)
            return t

        e = put(-1, "embed", model["embed"])
        self.lib.b200_decoder_set_tensor(self.handle, -1, T["lm_head"], e)
        put(-1, "final_norm", model["final_norm"])
        put(-1, "inv_freq", model["inv_freq"])
        for i, L in enumerate(model["layers"]):
            for name in T:
                if name in L and isinstance(L[name], np.ndarray):
                    put(i, name, L[name])

    def configure(self, fused, graph):
        self.lib.b200_decoder_configure(self.handle, int(fused), int(graph))

    def reset(self):
        self.lib.b200_decoder_reset(self.handle)

    def step_host(self, tokens):
        tokens = np.ascontiguousarray(tokens, np.int32)
        nxt = np.empty(self.batch, np.int32)
        self.lib.b200_decoder_step_host(self.handle, tokens.ctypes.data, nxt.ctypes.data)
        return nxt

    def prefill(self, tokens):
        """tokens [batch, T]: the whole prompt at once; returns the greedy picks."""
        import torch
        from gpu_util import dev
        tokens = np.ascontiguousarray(tokens, np.int32).reshape(self.batch, -1)
        t = dev(tokens)
        nxt = torch.empty(self.batch, dtype=torch.int32, device="cuda")
        self.lib.b200_decoder_prefill(self.handle, t, tokens.shape[1], nxt)
        self.lib.b200_synchronize()
        return nxt.cpu().numpy()

    def prefill_ragged(self, prompts):
        """prompts: one 1-D token array per sequence (different lengths); returns the picks."""
        import torch
        from gpu_util import dev
        assert len(prompts) == self.batch
        lengths = np.array([len(p) for p in prompts], np.int32)
        t = dev(np.concatenate([np.asarray(p, np.int32) for p in prompts]))
        nxt = torch.empty(self.batch, dtype=torch.int32, device="cuda")
        self.lib.b200_decoder_prefill_ragged(self.handle, t, lengths.ctypes.data, nxt)
        self.lib.b200_synchronize()
        return nxt.cpu().numpy()

    def logits(self):
        import torch
        p = C.c_void_p()
        self.lib.b200_decoder_logits(self.handle, C.byref(p))
        n = self.batch * self.cfg["vocab"]
        buf = torch.empty(n, dtype=torch.float32, device="cuda")
        self.lib.b200_copy(buf, 1, p.value, 1, n * 4)
        torch.cuda.synchronize()
        return buf.cpu().numpy().reshape(self.batch, self.cfg["vocab"])

    def set_sampling(self, cfg, seed=0):
        """cfg: oracle_lib.Sampling, or None for the greedy arg-max."""
        if cfg is None:
            self.lib.b200_decoder_set_sampling(self.handle, None)
        else:
            self.lib.b200_decoder_set_sampling(self.handle, C.byref(B200Sampling.of(cfg, seed)))

    def score_tokens(self, tokens, mask=None):
        tokens = np.ascontiguousarray(tokens, np.int32)
        m = None if mask is None else np.ascontiguousarray(mask, np.uint8)
        nll, n = C.c_double(), C.c_int64()
        self.lib.b200_decoder_score_tokens(self.handle, tokens.ctypes.data, tokens.size,
                                           None if m is None else m.ctypes.data, C.byref(nll), C.byref(n))
        return nll.value, n.value

    def launches(self):
        n = C.c_int()
        self.lib.b200_decoder_launches_per_step(self.handle, C.byref(n))
        return n.value

    def step_bytes(self):
        b = C.c_double()
        self.lib.b200_decoder_step_bytes(self.handle, C.byref(b))
        return b.value

    def close(self):
        if self.handle:
            self.lib.b200_decoder_destroy(self.handle)
            self.handle = None


# ---------------------------------------------------------------------------
# The same model through the reference engine's own Model + Generator
# ---------------------------------------------------------------------------
def ref_param_shapes(cfg):
    """Parameter names and shapes as the reference's Model allocates them
    (model/model.cpp:1087-1160)."""
    d, V = cfg["hidden"], cfg["vocab"]
    hd = cfg["head_dim"]
    qd, kvd = cfg["n_heads"] * hd, cfg["n_kv"] * hd
    ne, E, SH = cfg["n_experts"], cfg["expert_dim"], cfg["shared_dim"]
    d_inner = cfg["mamba_heads"] * cfg["mamba_d_head"]
    conv_dim = d_inner + 2 * cfg["mamba_d_state"]
    proj = d_inner + conv_dim + cfg["mamba_heads"]
    shapes = {"tok_embeddings": (V, d), "final_norm": (d,)}
    for i, t in enumerate(cfg["layer_types"]):
        p = f"layers.{i}."
        shapes[p + "attn_norm"] = (d,)
        shapes[p + "ffn_norm"] = (d,)
        if t == 0:
            shapes[p + "mamba.in_proj"] = (proj, d)
            shapes[p + "mamba.conv1d.weight"] = (conv_dim, cfg["mamba_d_conv"])
            shapes[p + "mamba.conv1d.bias"] = (conv_dim,)
            shapes[p + "mamba.dt_bias"] = (cfg["mamba_heads"],)
            shapes[p + "mamba.A_log"] = (cfg["mamba_heads"],)
            shapes[p + "mamba.D"] = (cfg["mamba_heads"],)
            shapes[p + "mamba.norm.weight"] = (d_inner,)
            shapes[p + "mamba.out_proj"] = (d, d_inner)
        else:
            shapes[p + "wq"] = (qd, d)
            shapes[p + "wk"] = (kvd, d)
            shapes[p + "wv"] = (kvd, d)
            shapes[p + "wo"] = (d, qd)
        shapes[p + "moe_router"] = (ne, d)
        shapes[p + "moe_gate"] = (ne * E, d)
        shapes[p + "moe_up"] = (ne * E, d)
        shapes[p + "moe_down"] = (ne * d, E)
        shapes[p + "moe_sh_gate"] = (SH, d)
        shapes[p + "moe_sh_up"] = (SH, d)
        shapes[p + "moe_sh_down"] = (d, SH)
    return shapes


def random_f32_params(cfg, seed=0, w_std=0.02):
    """fp32 source weights keyed by the reference's parameter names."""
    r = np.random.default_rng(seed)
    out = {}
    for name, shape in ref_param_shapes(cfg).items():
        n = int(np.prod(shape))
        leaf = name.split(".")[-1] if not name.endswith("norm.weight") else "norm.weight"
        if "norm" in name and "conv" not in name:
            a = 1 + 0.1 * r.standard_normal(n)
        elif leaf == "A_log":
            a = r.uniform(np.log(1.0), np.log(16.0), n)
        elif leaf == "dt_bias":
            a = np.log(np.expm1(r.uniform(1e-3, 1e-1, n)))
        elif leaf == "D":
            a = r.standard_normal(n)
        elif "conv1d" in name:
            a = r.standard_normal(n) * 0.1
        elif leaf == "moe_router":
            a = r.standard_normal(n) / np.sqrt(cfg["hidden"])
        else:
            a = r.standard_normal(n) * w_std
        out[name] = a.astype(np.float32).reshape(shape)
    return out


def model_from_f32(oracle, cfg, params):
    """The stored-form model (as make_model returns) from fp32 source weights, with
    the reference's storage policy: packed matrices, fp16 embeddings, fp32 the rest."""
    q = cfg["qkind"]
    hd = cfg["head_dim"]
    m = {"cfg": cfg, "layers": [], "embed": oracle.f32_to_f16(params["tok_embeddings"]),
         "final_norm": params["final_norm"],
         "inv_freq": (1.0 / cfg["rope_theta"] ** (np.arange(hd // 2) * 2.0 / hd)).astype(np.float32)}
    d_inner = cfg["mamba_heads"] * cfg["mamba_d_head"]
    conv_dim = d_inner + 2 * cfg["mamba_d_state"]
    for i, t in enumerate(cfg["layer_types"]):
        p = f"layers.{i}."
        L = {"type": t, "attn_norm": params[p + "attn_norm"], "ffn_norm": params[p + "ffn_norm"]}
        if t == 0:
            L.update(w_in=store_weight(oracle, params[p + "mamba.in_proj"], q),
                     conv_w=params[p + "mamba.conv1d.weight"], conv_b=params[p + "mamba.conv1d.bias"],
                     dt_bias=params[p + "mamba.dt_bias"], a_log=params[p + "mamba.A_log"], D=params[p + "mamba.D"],
                     norm_w=params[p + "mamba.norm.weight"], w_out=store_weight(oracle, params[p + "mamba.out_proj"], q),
                     d_inner=d_inner, conv_dim=conv_dim)
        else:
            for k in ("wq", "wk", "wv", "wo"):
                L[k] = store_weight(oracle, params[p + k], q)
        L["router"] = params[p + "moe_router"]
        L["router_bias"] = None
        for mine, theirs in (("gate", "moe_gate"), ("up", "moe_up"), ("down", "moe_down"), ("sh_gate", "moe_sh_gate"),
                             ("sh_up", "moe_sh_up"), ("sh_down", "moe_sh_down")):
            L[mine] = store_weight(oracle, params[p + theirs], q)
        m["layers"].append(L)
    return m


class RefGenerator:
    """The reference's Model + Generator behind oracle/_ref (lib: 'ref' = its CPU
    device, 'b200' = its CUDA device with this repository's backend linked in)."""

    def __init__(self, cfg, params, max_ctx, lib="ref"):
        import os
        from oracle_lib import ROOT
        path = os.path.join(ROOT, "oracle", "_ref", "libgai_ref.so" if lib == "ref" else "libgai_b200.so")
        self.lib = C.CDLL(path)
        self.lib.ref_model_create.restype = C.c_void_p
        self.lib.ref_last_error.restype = C.c_char_p
        self.cfg = cfg
        icfg = np.array([cfg["vocab"], cfg["hidden"], cfg["n_layers"], cfg["n_heads"], cfg["n_kv"], cfg["head_dim"],
                         cfg["rope_type"], cfg["mamba_heads"], cfg["mamba_d_head"], cfg["mamba_d_state"],
                         cfg["mamba_d_conv"], cfg["n_experts"], cfg["top_k"], cfg["expert_dim"], cfg["shared_dim"],
                         max(max_ctx, 64)], np.int32)
        fcfg = np.array([cfg["rope_theta"], cfg["rms_eps"], cfg["embedding_multiplier"], cfg["residual_multiplier"],
                         cfg["attn_scale"], cfg["logits_scaling"]], np.float32)
        types = np.array(cfg["layer_types"], np.int32)
        self.h = self.lib.ref_model_create(icfg.ctypes.data_as(C.c_void_p), fcfg.ctypes.data_as(C.c_void_p),
                                           types.ctypes.data_as(C.c_void_p), 0 if lib == "ref" else 1,
                                           cfg["qkind"])
        if not self.h:
            raise RuntimeError("ref_model_create: " + self.lib.ref_last_error().decode())
        self.h = C.c_void_p(self.h)
        for name, a in params.items():
            a = np.ascontiguousarray(a, np.float32)
            self._ck(self.lib.ref_model_set_param(self.h, name.encode(), a.ctypes.data_as(C.c_void_p),
                                                  C.c_int64(a.size)), name)
        self._ck(self.lib.ref_generator_create(self.h, max_ctx), "generator")
        self.pos = 0

    def _ck(self, rc, what):
        if rc != 0:
            raise RuntimeError(f"{what}: " + self.lib.ref_last_error().decode())

    def step(self, token):
        out = np.empty(self.cfg["vocab"], np.float32)
        self._ck(self.lib.ref_decode_step(self.h, int(token), self.pos, out.ctypes.data_as(C.c_void_p)), "decode_step")
        self.pos += 1
        return out

    def score_tokens(self, tokens, mask=None):
        """Generator::score_tokens: (mean negative log-likelihood, scored tokens)."""
        tokens = np.ascontiguousarray(tokens, np.int32)
        m = None if mask is None else np.ascontiguousarray(mask, np.uint8)
        nll, n = C.c_double(), C.c_int64()
        self._ck(self.lib.ref_score_tokens(self.h, tokens.ctypes.data_as(C.c_void_p), tokens.size,
                                           None if m is None else m.ctypes.data_as(C.c_void_p), C.byref(nll), C.byref(n)),
                 "score_tokens")
        return nll.value, n.value

    def generate(self, prompt, max_new, sampling, seed):
        """Generator::prefill + generate with an oracle_lib.Sampling configuration."""
        prompt = np.ascontiguousarray(prompt, np.int32)
        out = np.empty(max_new, np.int32)
        n = C.c_int()
        self._ck(self.lib.ref_generate(self.h, prompt.ctypes.data_as(C.c_void_p), prompt.size, max_new,
                                       sampling.f.ctypes.data_as(C.c_void_p), sampling.i.ctypes.data_as(C.c_void_p),
                                       C.c_uint64(seed), out.ctypes.data_as(C.c_void_p), C.byref(n)), "generate")
        return out[:n.value].copy()

    def close(self):
        if self.h:
            self.lib.ref_model_destroy(self.h)
            self.h = None
