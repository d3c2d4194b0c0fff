"""ctypes front-ends for the two CPU checkers (test infrastructure).

`Oracle` wraps oracle/liboracle.so (the scalar restatement); `Ref` wraps
oracle/_ref/libgai_ref.so (the reference engine's own CPU objects behind an
extern "C" bridge) and is only available where that library was built.  Both
expose the same method names and numpy in / numpy out, so a test can run either.
"""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_SO = os.path.join(ROOT, "oracle", "liboracle.so")
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libgai_ref.so")

BLOCK_ELEMS = {0: 32, 1: 32, 2: 32, 3: 256, 4: 32}
BLOCK_BYTES = {0: 18, 1: 20, 2: 34, 3: 144, 4: 18}
KIND_NAMES = {0: "q4_0", 1: "q4_1", 2: "q8_0", 3: "q4_k"}


def packed_bytes(kind, n):
    be = BLOCK_ELEMS[kind]
    return (n + be - 1) // be * BLOCK_BYTES[kind]


def build_oracle():
    """Compile liboracle.so (and _ref when the reference sources are mounted)."""
    subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "-j8"], check=True,
                   stdout=subprocess.DEVNULL)


def _p(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle buffers must be contiguous"
    return a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.int32)


def _wt(w, wkind):
    """Weights travel as raw bytes: fp32 array, uint16 (fp16 bits) array or packed uint8."""
    if w is None:
        return None
    want = {-2: np.float32, -1: np.uint16}.get(wkind, np.uint8)
    a = np.ascontiguousarray(w)
    assert a.dtype == want, f"weight dtype {a.dtype} does not match wkind {wkind}"
    return a


class Sampling:
    """SamplingConfig (inference/sampler.h:9-24) as the two packed arrays the checkers take."""

    def __init__(self, temperature=0.8, top_k=40, top_p=0.92, min_p=0.05, repetition_penalty=1.12,
                 repetition_window=128, frequency_penalty=0.0, presence_penalty=0.0, no_repeat_ngram=0, greedy=False):
        self.f = np.array([temperature, top_p, min_p, repetition_penalty, frequency_penalty, presence_penalty], np.float32)
        self.i = np.array([top_k, repetition_window, no_repeat_ngram, int(greedy)], np.int32)

    temperature = property(lambda s: float(s.f[0]))
    top_p = property(lambda s: float(s.f[1]))
    min_p = property(lambda s: float(s.f[2]))
    repetition_penalty = property(lambda s: float(s.f[3]))
    frequency_penalty = property(lambda s: float(s.f[4]))
    presence_penalty = property(lambda s: float(s.f[5]))
    top_k = property(lambda s: int(s.i[0]))
    repetition_window = property(lambda s: int(s.i[1]))
    no_repeat_ngram = property(lambda s: int(s.i[2]))
    greedy = property(lambda s: bool(s.i[3]))

    def copy(self):
        c = Sampling()
        c.f, c.i = self.f.copy(), self.i.copy()
        return c


class _Base:
    prefix = ""

    def __init__(self, path):
        self.lib = C.CDLL(path)

    def fn(self, name):
        return getattr(self.lib, self.prefix + name)

    def _call(self, name, *args):
        rc = self.fn(name)(*args)
        if rc not in (0, None):
            raise ValueError(f"{self.prefix}{name} failed: {self.error()}")

    def error(self):
        return "rc != 0"


class Oracle(_Base):
    prefix = "ora_"

    def __init__(self):
        if not os.path.exists(ORACLE_SO):
            build_oracle()
        super().__init__(ORACLE_SO)
        self.lib.ora_argmax.restype = C.c_int32
        self.lib.ora_sample.restype = C.c_int32
        self.lib.ora_sample_candidates.restype = C.c_int32
        self.lib.ora_rng_uniform.restype = C.c_float
        self.lib.ora_rng_next.restype = C.c_uint64
        for n in ("rng_seed", "sampling_validate", "softmax_cross_entropy"):
            self.fn(n).restype = None
        self.lib.ora_packed_bytes.restype = C.c_int64
        for n in ("f32_to_f16", "f16_to_f32", "dequantize", "dequantize_f32", "linear_f16",
                  "linear_f32", "embedding", "rmsnorm", "rope_cached", "swiglu", "topk",
                  "rep_penalties", "moe_route", "moe_permutation", "attention_forward"):
            self.fn(n).restype = None

    # --- formats -----------------------------------------------------------
    def f32_to_f16(self, x):
        x = _f32(x)
        out = np.empty(x.shape, np.uint16)
        self.lib.ora_f32_to_f16(_p(x), _p(out), C.c_int64(x.size))
        return out

    def f16_to_f32(self, h):
        h = np.ascontiguousarray(h, dtype=np.uint16)
        out = np.empty(h.shape, np.float32)
        self.lib.ora_f16_to_f32(_p(h), _p(out), C.c_int64(h.size))
        return out

    def quantize(self, x, kind):
        x = _f32(x)
        out = np.zeros(packed_bytes(kind, x.size), np.uint8)
        self._call("quantize", _p(x), _p(out), C.c_int64(x.size), kind)
        return out

    def dequantize(self, packed, n, kind):
        out = np.empty(n, np.uint16)
        self.lib.ora_dequantize(_p(packed), _p(out), C.c_int64(n), kind)
        return out

    def dequantize_f32(self, packed, n, kind):
        out = np.empty(n, np.float32)
        self.lib.ora_dequantize_f32(_p(packed), _p(out), C.c_int64(n), kind)
        return out

    # --- linears -----------------------------------------------------------
    def linear(self, x, w, wkind, M, K, N):
        x = _f32(x)
        w = _wt(w, wkind)
        y = np.empty((M, N), np.float32)
        self._call("linear_any", _p(x), _p(w), wkind, _p(y), M, K, N)
        return y

    def set_weight_rounding(self, on):
        """True (default): linear layers use fp16-rounded dequantised weights like the
        reference's CPU path; False: the exact dequantised values like its CUDA path."""
        self.lib.ora_set_weight_rounding(int(bool(on)))

    def linear_exact(self, x, w, kind, M, K, N):
        """Packed weights without the fp16 rounding of each weight, double accumulation."""
        x = _f32(x)
        w = _wt(w, kind)
        y = np.empty((M, N), np.float32)
        self._call("linear_q4_exact", _p(x), _p(w), _p(y), M, K, N, kind)
        return y

    # --- small ops ---------------------------------------------------------
    def embedding(self, ids, table, half, dim, vocab):
        ids = _i32(ids)
        out = np.empty((ids.size, dim), np.float32)
        self.fn("embedding")(_p(ids), _p(table), int(half), _p(out), C.c_int64(ids.size), dim, vocab)
        return out

    def rmsnorm(self, x, w, eps, want_rrms=False):
        x = _f32(x)
        rows, dim = x.shape
        out = np.empty_like(x)
        rr = np.empty(rows, np.float32) if want_rrms else None
        self.fn("rmsnorm")(_p(x), _p(_f32(w)), _p(out), _p(rr), C.c_int64(rows), dim, C.c_float(eps))
        return (out, rr) if want_rrms else out

    def rope_cached(self, q, k, pos, inv_freq, n_heads, n_kv, head_dim, rope_type):
        q = None if q is None else _f32(q).copy()
        k = None if k is None else _f32(k).copy()
        pos = _i32(pos)
        self.fn("rope_cached")(_p(q), _p(k), _p(pos), _p(_f32(inv_freq)), C.c_int64(pos.size),
                               n_heads, n_kv, head_dim, rope_type)
        return q, k

    def swiglu(self, g, u):
        g, u = _f32(g), _f32(u)
        out = np.empty_like(g)
        self.fn("swiglu")(_p(g), _p(u), _p(out), C.c_int64(g.size))
        return out

    def argmax(self, logits):
        logits = _f32(logits)
        return int(self.lib.ora_argmax(_p(logits), logits.size))

    def topk(self, logits, K):
        logits = _f32(logits)
        vals = np.empty(K, np.float32)
        ids = np.empty(K, np.int32)
        self.fn("topk")(_p(logits), logits.size, K, _p(vals), _p(ids))
        return vals, ids

    def rep_penalties(self, logits, hist, rep, freq, pres):
        logits = _f32(logits).copy()
        hist = _i32(hist)
        self.fn("rep_penalties")(_p(logits), logits.size, _p(hist), hist.size, C.c_float(rep),
                                 C.c_float(freq), C.c_float(pres))
        return logits

    # --- sampling tail -------------------------------------------------------
    def rng_state(self, seed):
        st = np.zeros(4, np.uint64)
        self.lib.ora_rng_seed(C.c_uint64(seed), _p(st))
        return st

    def rng_uniform(self, seed, n):
        st = self.rng_state(seed)
        return np.array([self.lib.ora_rng_uniform(_p(st)) for _ in range(n)], np.float32)

    def sampling_validate(self, cfg):
        c = cfg.copy()
        self.fn("sampling_validate")(_p(c.f), _p(c.i))
        return c

    def sample_with_state(self, logits, hist, cfg, state):
        """One Sampler::sample call; `logits` (modified in place) and `state` advance."""
        hist = _i32(hist if hist is not None else [])
        return int(self.lib.ora_sample(_p(logits), logits.size, _p(hist), hist.size, _p(cfg.f), _p(cfg.i), _p(state)))

    def sample(self, logits, hist, cfg, seed, n_draws):
        st = self.rng_state(seed)
        logits = _f32(logits)
        return np.array([self.sample_with_state(logits.copy(), hist, cfg, st) for _ in range(n_draws)], np.int32)

    def candidates_with_state(self, vals, ids, cfg, state):
        vals, ids = _f32(vals), _i32(ids)
        return int(self.lib.ora_sample_candidates(_p(vals), _p(ids), vals.size, C.c_float(cfg.temperature),
                                                  C.c_float(cfg.top_p), C.c_float(cfg.min_p), _p(state)))

    def sample_candidates(self, vals, ids, cfg, seed, n_draws):
        st = self.rng_state(seed)
        return np.array([self.candidates_with_state(vals, ids, cfg, st) for _ in range(n_draws)], np.int32)

    def cross_entropy(self, logits, targets, z_scale=0.0):
        logits, targets = _f32(logits), _i32(targets)
        n, V = logits.shape
        total, count = C.c_double(), C.c_int64()
        self.fn("softmax_cross_entropy")(_p(logits), _p(targets), C.c_int64(n), V, C.c_float(z_scale), C.byref(total),
                                         C.byref(count))
        return total.value, count.value

    # --- MoE ---------------------------------------------------------------
    def moe_route(self, x, router_w, router_bias, ne, K):
        x = _f32(x)
        N, d = x.shape
        probs = np.empty((N, ne), np.float32)
        idx = np.empty((N, K), np.int32)
        w = np.empty((N, K), np.float32)
        self.fn("moe_route")(_p(x), _p(_f32(router_w)), _p(_f32(router_bias)), _p(probs), _p(idx),
                             _p(w), C.c_int64(N), d, ne, K)
        return probs, idx, w

    def moe_permutation(self, idx, ne):
        idx = _i32(idx).reshape(-1)
        grouped = np.empty(idx.size, np.int32)
        offsets = np.empty(ne + 1, np.int32)
        self.fn("moe_permutation")(_p(idx), C.c_int64(idx.size), ne, _p(grouped), _p(offsets))
        return grouped, offsets

    def moe_forward(self, x, router_w, router_bias, gates, ups, downs, sh_g, sh_u, sh_d,
                    d, E, ne, K, SH, wkind):
        x = _f32(x)
        N = x.shape[0]
        out = np.empty((N, d), np.float32)
        probs = np.empty((N, ne), np.float32)
        idx = np.empty((N, K), np.int32)
        w = np.empty((N, K), np.float32)
        ws = [_wt(a, wkind) for a in (gates, ups, downs, sh_g, sh_u, sh_d)]
        self._call("moe_forward", _p(x), _p(_f32(router_w)), _p(_f32(router_bias)),
                   *[_p(a) for a in ws], _p(out), _p(probs), _p(idx), _p(w), C.c_int64(N),
                   d, E, ne, K, SH, wkind)
        return out, probs, idx, w

    # --- Mamba-2 -----------------------------------------------------------
    def mamba2_forward(self, x, w_in, conv_w, conv_b, dt_bias, a_log, D, norm_w, w_out, state,
                       B, T, d, d_inner, conv_dim, n_heads, d_head, d_state, k, eps, wkind):
        x = _f32(x)
        state = _f32(state).copy()
        out = np.empty((B, T, d), np.float32)
        self._call("mamba2_forward", _p(x), _p(_wt(w_in, wkind)), _p(_f32(conv_w)),
                   _p(_f32(conv_b)), _p(_f32(dt_bias)), _p(_f32(a_log)), _p(_f32(D)),
                   _p(_f32(norm_w)), _p(_wt(w_out, wkind)), _p(state), _p(out), B, T, d, d_inner,
                   conv_dim, n_heads, d_head, d_state, k, C.c_float(eps), wkind)
        return out, state

    # --- attention ---------------------------------------------------------
    def attention_forward(self, q, k, v, B, T, H, KV, hd, scale, window=0, segment_ids=None,
                          want_probs=False):
        q, k, v = _f32(q), _f32(k), _f32(v)
        out = np.empty((B, T, H, hd), np.float32)
        probs = np.empty((B, H, T, T), np.float32) if want_probs else None
        seg = _i32(segment_ids)
        r = self.fn("attention_forward")(_p(q), _p(k), _p(v), _p(out), _p(probs), B, T, H, KV, hd,
                                         C.c_float(scale), window, _p(seg))
        if r not in (0, None):
            raise ValueError(self.error())
        return (out, probs) if want_probs else out

    def attention_decode_ring(self, q, kc, vc, half, H, KV, hd, ring_start, pinned, cur_len,
                              cache_max, scale, window=0):
        q = _f32(q)
        out = np.empty((H, hd), np.float32)
        self._call("attention_decode_ring", _p(q), _p(kc), _p(vc), int(half), _p(out), H, KV, hd,
                   ring_start, pinned, cur_len, cache_max, C.c_float(scale), window)
        return out

    def num_threads(self):
        return int(self.fn("num_threads")())


class OracleOnly(Oracle):
    """Functions that only the restatement has (no counterpart callable in the reference)."""

    def mamba2_core(self, proj, conv_w, conv_b, dt_bias, a_log, D, norm_w, conv_state, state,
                    B, T, d_inner, conv_dim, n_heads, d_head, d_state, k, eps):
        proj = _f32(proj)
        state = _f32(state).copy()
        conv_state = None if conv_state is None else _f32(conv_state).copy()
        normed = np.empty((B * T, d_inner), np.float32)
        self._call("mamba2_core", _p(proj), _p(_f32(conv_w)), _p(_f32(conv_b)), _p(_f32(dt_bias)),
                   _p(_f32(a_log)), _p(_f32(D)), _p(_f32(norm_w)), _p(conv_state), _p(state),
                   _p(normed), B, T, d_inner, conv_dim, n_heads, d_head, d_state, k,
                   C.c_float(eps))
        return normed, conv_state, state

    def mamba2_step(self, x, w_in, conv_w, conv_b, dt_bias, a_log, D, norm_w, w_out, conv_state,
                    ssm_state, d, d_inner, conv_dim, n_heads, d_head, d_state, k, eps, wkind):
        x = _f32(x)
        conv_state = _f32(conv_state).copy()
        ssm_state = _f32(ssm_state).copy()
        out = np.empty(d, np.float32)
        self._call("mamba2_step", _p(x), _p(_wt(w_in, wkind)), _p(_f32(conv_w)), _p(_f32(conv_b)),
                   _p(_f32(dt_bias)), _p(_f32(a_log)), _p(_f32(D)), _p(_f32(norm_w)),
                   _p(_wt(w_out, wkind)), _p(conv_state), _p(ssm_state), _p(out), d, d_inner,
                   conv_dim, n_heads, d_head, d_state, k, C.c_float(eps), wkind)
        return out, conv_state, ssm_state


class Ref(Oracle):
    """The reference engine's CPU objects.  Same method names as `Oracle`; Q4_K
    (kind 3), K > 8 and ne > 64 are not available here (the reference rejects them)."""
    prefix = "ref_"

    def __init__(self):
        if not os.path.exists(REF_SO):
            raise FileNotFoundError(REF_SO)
        _Base.__init__(self, REF_SO)
        self.lib.ref_last_error.restype = C.c_char_p

    @staticmethod
    def available():
        return os.path.exists(REF_SO)

    def error(self):
        return self.lib.ref_last_error().decode()

    def quantize(self, x, kind):
        x = _f32(x)
        out = np.zeros(packed_bytes(kind, x.size), np.uint8)
        self._call("quantize", _p(x), _p(out), C.c_int64(x.size), kind)
        return out

    def dequantize(self, packed, n, kind):
        out = np.empty(n, np.uint16)
        self._call("quant_materialize", _p(packed), _p(out), C.c_int64(n), kind)
        return out

    def dequantize_f32(self, packed, n, kind):
        out = np.empty(n, np.float32)
        self._call("dequantize_f32", _p(packed), _p(out), C.c_int64(n), kind)
        return out

    def linear(self, x, w, wkind, M, K, N):
        x = _f32(x)
        w = _wt(w, wkind)
        y = np.empty((M, N), np.float32)
        if wkind == -2:
            self._call("linear_f32", _p(x), _p(w), _p(y), M, K, N)
        elif wkind == -1:
            self._call("linear_f16", _p(x), _p(w), _p(y), M, K, N)
        else:
            self._call("linear_q4", _p(x), _p(w), _p(y), M, K, N, wkind)
        return y

    def argmax(self, logits):
        logits = _f32(logits)
        out = C.c_int32(0)
        self._call("argmax", _p(logits), logits.size, C.byref(out))
        return out.value

    def rng_uniform(self, seed, n):
        out = np.empty(n, np.float32)
        self._call("rng_uniform", C.c_uint64(seed), n, _p(out))
        return out

    def sampling_validate(self, cfg):
        c = cfg.copy()
        self._call("sampling_validate", _p(c.f), _p(c.i))
        return c

    def sample(self, logits, hist, cfg, seed, n_draws):
        logits, hist = _f32(logits), _i32(hist if hist is not None else [])
        out = np.empty(n_draws, np.int32)
        self._call("sampler_sample", _p(logits), logits.size, _p(hist), hist.size, _p(cfg.f), _p(cfg.i),
                   C.c_uint64(seed), n_draws, _p(out))
        return out

    def sample_candidates(self, vals, ids, cfg, seed, n_draws):
        vals, ids = _f32(vals), _i32(ids)
        out = np.empty(n_draws, np.int32)
        self._call("sampler_candidates", _p(vals), _p(ids), vals.size, _p(cfg.f), _p(cfg.i), C.c_uint64(seed), n_draws,
                   _p(out))
        return out

    def cross_entropy(self, logits, targets, z_scale=0.0):
        logits, targets = _f32(logits), _i32(targets)
        n, V = logits.shape
        total, count = C.c_double(), C.c_int64()
        self._call("softmax_cross_entropy", _p(logits), _p(targets), C.c_int64(n), V, C.c_float(z_scale),
                   C.byref(total), C.byref(count))
        return total.value, count.value

    def moe_route(self, x, router_w, router_bias, ne, K):
        raise NotImplementedError("the reference exposes routing only through moe_forward")

    def moe_permutation(self, idx, ne):
        raise NotImplementedError("the reference CPU path has no permutation")
