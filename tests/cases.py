"""Seeded synthetic inputs shared by the CPU and GPU tests.

Distributions follow the workload description the benchmark is quoted on: linear
weights N(0, 0.02) then quantised, A_log ~ U(log 1, log 16), dt_bias =
softplus^-1(U(1e-3, 1e-1)), D ~ N(0, 1), conv weights N(0, 0.1), router weights
N(0, 1/d) so router logits are ~N(0, 1), router bias N(0, sigma).
"""
import numpy as np


def store_weight(oracle, w_f32, wkind):
    """fp32 matrix -> the storage form named by wkind (-2 fp32, -1 fp16 bits, 0..3 packed)."""
    w_f32 = np.ascontiguousarray(w_f32, dtype=np.float32)
    if wkind == -2:
        return w_f32
    if wkind == -1:
        return oracle.f32_to_f16(w_f32)
    return oracle.quantize(w_f32.reshape(-1), wkind)


def moe_case(oracle, seed, N, d, E, ne, K, SH, wkind, bias_sigma=None, x_scale=1.0):
    r = np.random.default_rng(seed)
    c = {
        "x": (r.standard_normal((N, d)) * x_scale).astype(np.float32),
        "router_w": (r.standard_normal((ne, d)) / np.sqrt(d)).astype(np.float32),
    }
    if bias_sigma is None:
        bias_sigma = 0.5 / ne
    c["router_bias"] = (r.standard_normal(ne) * bias_sigma).astype(np.float32) if bias_sigma > 0 else None
    c["gates"] = store_weight(oracle, r.standard_normal((ne * E, d)) * 0.02, wkind)
    c["ups"] = store_weight(oracle, r.standard_normal((ne * E, d)) * 0.02, wkind)
    c["downs"] = store_weight(oracle, r.standard_normal((ne * d, E)) * 0.02, wkind)
    if SH > 0:
        c["sh_g"] = store_weight(oracle, r.standard_normal((SH, d)) * 0.02, wkind)
        c["sh_u"] = store_weight(oracle, r.standard_normal((SH, d)) * 0.02, wkind)
        c["sh_d"] = store_weight(oracle, r.standard_normal((d, SH)) * 0.02, wkind)
    else:
        c["sh_g"] = c["sh_u"] = c["sh_d"] = None
    return c


def mamba_params(oracle, r, d, n_heads, d_head, d_state, k, wkind, w_std=0.02):
    d_inner = n_heads * d_head
    conv_dim = d_inner + 2 * d_state
    proj = d_inner + conv_dim + n_heads
    u = r.uniform(1e-3, 1e-1, n_heads)
    p = {
        "w_in": store_weight(oracle, r.standard_normal((proj, d)) * w_std, wkind),
        "conv_w": (r.standard_normal((conv_dim, k)) * 0.1).astype(np.float32),
        "conv_b": (r.standard_normal(conv_dim) * 0.1).astype(np.float32),
        "dt_bias": np.log(np.expm1(u)).astype(np.float32),
        "a_log": r.uniform(np.log(1.0), np.log(16.0), n_heads).astype(np.float32),
        "D": r.standard_normal(n_heads).astype(np.float32),
        "norm_w": (1.0 + 0.1 * r.standard_normal(d_inner)).astype(np.float32),
        "w_out": store_weight(oracle, r.standard_normal((d, d_inner)) * w_std, wkind),
        "d_inner": d_inner, "conv_dim": conv_dim, "proj": proj,
    }
    return p


def mamba_case(oracle, seed, B, T, d, n_heads, d_head, d_state, k, wkind, w_std=0.2):
    """w_std defaults to a large value so the projected activations are O(1) at tiny d."""
    r = np.random.default_rng(seed)
    p = mamba_params(oracle, r, d, n_heads, d_head, d_state, k, wkind, w_std)
    x = r.standard_normal((B, T, d)).astype(np.float32)
    state = (r.standard_normal((B, n_heads, d_head, d_state)) * 0.1).astype(np.float32)
    args = (x, p["w_in"], p["conv_w"], p["conv_b"], p["dt_bias"], p["a_log"], p["D"], p["norm_w"],
            p["w_out"], state, B, T, d, p["d_inner"], p["conv_dim"], n_heads, d_head, d_state, k,
            1e-5)
    return {"args": args, "params": p}
