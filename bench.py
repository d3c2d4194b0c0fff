#!/usr/bin/env python
"""Decode-throughput benchmark of the quantized hybrid-layer forward step.

Workload (N = 1): the Granite-4.0-H-Tiny-shaped model - hidden 1536, vocab 100352,
40 layers (36 Mamba-2: 48 heads x 64, d_state 128, conv 4; 4 GQA at layers
9/19/29/39: 12 q / 4 kv heads, head_dim 128, no RoPE), MoE with 64 experts, top-6,
expert ffn 512, shared expert 1024 - with random-init N(0, 0.02) weights quantised
to Q4_K on the device, batch 1, greedy decode after a `--ctx`-token prompt.
One step = one decoded token per sequence.

    value         tok/s with the token ids resident on the device (the step is one
                  CUDA graph; CUDA events on the launching stream)
    e2e           tok/s through b200_decoder_step_host: host token id in, host
                  arg-max out, a stream synchronise per token
    roofline      achieved HBM GB/s of the whole step and of its dominant kernel
                  against the measured copy bandwidth
    cpu_baseline  the reference engine's CPU ops (oracle/_ref) or the oracle port on
                  this box's host cores, on a bounded sample of the same token
    cpu_baseline_fp32  the same sample with fp32 weights (no per-call dequantisation): the
                  reference CPU path at its best
    prefill       the `--ctx`-token prompt through b200_decoder_prefill (tok/s, device time)
    moe_layer     one MoE layer of this shape over 4096 tokens (tensor-core grouped GEMM;
                  expert-parallel over NCCL all-to-all when N > 1); moe_sweep: the same layer
                  at 1 / 64 / 512 / 4096 tokens with the roofline that bounds each size
    batch64       64 sequences decoded together after a 4096-token prompt each (the prompt
                  of 64 x 4096 tokens through b200_decoder_prefill is timed as well)
    mamba_ops     Mamba-2 at the op level: the chunked SSD scan over [8, 4096, 48, 64] with
                  d_state 128, and the batch-64 single-token state update

`--only gemm` times the many-token kernels alone (also the small profiling case).

`--impl reference` prints the CPU arm alone.  Under torchrun (N > 1) every rank runs
an independent replica of the model (only the MoE layer shards in this workload and
expert parallelism is a separate mode), value is the sum over ranks.
"""
import argparse
import ctypes as C
import importlib
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

PKG = "jdm-ghassan_v1_flach_b200"

H_TINY = dict(vocab=100352, hidden=1536, n_layers=40,
              layer_types=[1 if l in (9, 19, 29, 39) else 0 for l in range(40)],
              n_heads=12, n_kv=4, head_dim=128, rope_type=-1, rope_theta=1e4,
              mamba_heads=48, mamba_d_head=64, mamba_d_state=128, mamba_d_conv=4,
              n_experts=64, top_k=6, expert_dim=512, shared_dim=1024, qkind=3,
              rms_eps=1e-5, embedding_multiplier=12.0, residual_multiplier=0.22,
              attn_scale=0.0078125, logits_scaling=6.0)

H_SMALL = dict(vocab=100352, hidden=4096, n_layers=40,
               layer_types=[1 if l in (9, 19, 29, 39) else 0 for l in range(40)],
               n_heads=32, n_kv=8, head_dim=128, rope_type=-1, rope_theta=1e4,
               mamba_heads=128, mamba_d_head=64, mamba_d_state=128, mamba_d_conv=4,
               n_experts=72, top_k=10, expert_dim=768, shared_dim=1536, qkind=3,
               rms_eps=1e-5, embedding_multiplier=12.0, residual_multiplier=0.22,
               attn_scale=0.0078125, logits_scaling=16.0)

T_IDS = dict(embed=0, final_norm=1, lm_head=2, inv_freq=3, attn_norm=10, ffn_norm=11,
             w_in=20, conv_w=21, conv_b=22, dt_bias=23, a_log=24, D=25, norm_w=26, w_out=27,
             wq=30, wk=31, wv=32, wo=33, router=40, router_bias=41, gate=42, up=43, down=44,
             sh_gate=45, sh_up=46, sh_down=47)


def measured_step_traffic(launches_per_step):
    """DRAM bytes (read + written) of one decode step of the default workload, from the
    committed ncu summary of that step: the summary carries a line
    `traffic_bytes_per_step: <bytes> launches_per_step: <n>`; the figure is used only while the
    step still has that many launches (null otherwise: the capture is then out of date)."""
    import re
    path = os.path.join(ROOT, "profiles", "decode_step_htiny_q4k_bs1_dram_bytes.md")
    try:
        m = re.search(r"traffic_bytes_per_step:\s*([0-9.eE+]+)\s+launches_per_step:\s*(\d+)", open(path).read())
    except OSError:
        return None
    if not m or int(m.group(2)) != int(launches_per_step):
        return None
    return float(m.group(1))


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ---------------------------------------------------------------------------
# model construction on the device
# ---------------------------------------------------------------------------
class DeviceModel:
    """Random-init weights generated and quantised on the GPU, bound to a b200_decoder."""

    def __init__(self, cfg, batch, max_ctx, seed=0, kv_page=64):
        import torch
        self.torch = torch
        self.lib = importlib.import_module(PKG).lib()
        self.cfg, self.batch = cfg, batch
        self.gen = torch.Generator(device="cuda").manual_seed(seed)
        self.tensors = {}
        c = cfg
        self.handle = C.c_void_p()
        types = np.array(c["layer_types"], np.int32)
        self.lib.b200_decoder_create(C.byref(self.handle), batch, c["vocab"], c["hidden"], c["n_layers"],
                                     types.ctypes.data, c["n_heads"], c["n_kv"], c["head_dim"], c["rope_type"],
                                     c["mamba_heads"], c["mamba_d_head"], c["mamba_d_state"], c["mamba_d_conv"],
                                     c["n_experts"], c["top_k"], c["expert_dim"], c["shared_dim"], max_ctx, kv_page,
                                     c["qkind"], c["rms_eps"], c["embedding_multiplier"], c["residual_multiplier"],
                                     c["attn_scale"], c["logits_scaling"])
        d, q = c["hidden"], c["qkind"]
        hd = c["head_dim"]
        qd, kvd = c["n_heads"] * hd, c["n_kv"] * hd
        ne, E, SH = c["n_experts"], c["expert_dim"], c["shared_dim"]
        d_inner = c["mamba_heads"] * c["mamba_d_head"]
        conv_dim = d_inner + 2 * c["mamba_d_state"]
        proj = d_inner + conv_dim + c["mamba_heads"]
        emb = (self.randn(c["vocab"] * d) * 0.02).half()
        self.put(-1, "embed", emb)
        self.lib.b200_decoder_set_tensor(self.handle, -1, T_IDS["lm_head"], emb)     # tied
        self.put(-1, "final_norm", 1 + 0.1 * self.randn(d))
        if c["rope_type"] >= 0:
            inv = 1.0 / c["rope_theta"] ** (torch.arange(hd // 2, device="cuda") * 2.0 / hd)
            self.put(-1, "inv_freq", inv.float())
        for l, t in enumerate(c["layer_types"]):
            self.put(l, "attn_norm", 1 + 0.1 * self.randn(d))
            self.put(l, "ffn_norm", 1 + 0.1 * self.randn(d))
            if t == 0:
                nh = c["mamba_heads"]
                self.put(l, "w_in", self.packed(proj * d))
                self.put(l, "conv_w", self.randn(conv_dim * c["mamba_d_conv"]) * 0.1)
                self.put(l, "conv_b", self.randn(conv_dim) * 0.1)
                u = torch.rand(nh, device="cuda", generator=self.gen) * (1e-1 - 1e-3) + 1e-3
                self.put(l, "dt_bias", torch.log(torch.expm1(u)))
                a = torch.rand(nh, device="cuda", generator=self.gen) * np.log(16.0)
                self.put(l, "a_log", a)
                self.put(l, "D", self.randn(nh))
                self.put(l, "norm_w", 1 + 0.1 * self.randn(d_inner))
                self.put(l, "w_out", self.packed(d * d_inner))
            else:
                self.put(l, "wq", self.packed(qd * d))
                self.put(l, "wk", self.packed(kvd * d))
                self.put(l, "wv", self.packed(kvd * d))
                self.put(l, "wo", self.packed(d * qd))
            self.put(l, "router", self.randn(ne * d) / np.sqrt(d))
            self.put(l, "router_bias", self.randn(ne) * 0.5 / ne)
            self.put(l, "gate", self.packed(ne * E * d))
            self.put(l, "up", self.packed(ne * E * d))
            self.put(l, "down", self.packed(ne * d * E))
            self.put(l, "sh_gate", self.packed(SH * d))
            self.put(l, "sh_up", self.packed(SH * d))
            self.put(l, "sh_down", self.packed(d * SH))
        torch.cuda.synchronize()

    def randn(self, n):
        return self.torch.randn(n, device="cuda", generator=self.gen, dtype=self.torch.float32)

    def packed(self, n, std=0.02):
        """N(0, std) weights in the model's storage: packed blocks, or fp16 when qkind is -1."""
        torch = self.torch
        q = self.cfg["qkind"]
        w = self.randn(n) * std
        if q < 0:
            return w.half()
        be, bb = (256, 144) if q == 3 else (32, {0: 18, 1: 20, 2: 34}[q])
        out = torch.empty(n // be * bb, dtype=torch.uint8, device="cuda")
        self.lib.b200_quantize(w, out, n, q)
        return out

    def put(self, layer, name, t):
        t = t.contiguous()
        self.tensors[(layer, name)] = t
        self.lib.b200_decoder_set_tensor(self.handle, layer, T_IDS[name], t)

    def configure(self, fused, graph):
        self.lib.b200_decoder_configure(self.handle, int(fused), int(graph))

    def step_dev(self, tok_dev):
        self.lib.b200_decoder_step(self.handle, tok_dev, tok_dev)       # in place: next token feeds the next step

    def prefill(self, prompt_dev, next_dev):
        """prompt_dev [batch, T] int32 on the device: the whole prompt through the many-token kernels."""
        self.lib.b200_decoder_prefill(self.handle, prompt_dev, int(prompt_dev.shape[1]), next_dev)

    def reset(self):
        self.lib.b200_decoder_reset(self.handle)

    def step_host(self, tok_np, out_np):
        self.lib.b200_decoder_step_host(self.handle, tok_np.ctypes.data, out_np.ctypes.data)

    def step_bytes(self):
        b = C.c_double()
        self.lib.b200_decoder_step_bytes(self.handle, C.byref(b))
        return b.value

    def launches(self):
        n = C.c_int()
        self.lib.b200_decoder_launches_per_step(self.handle, C.byref(n))
        return n.value

    def close(self):
        self.lib.b200_decoder_destroy(self.handle)


# ---------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi samples of this rank's GPU while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.path = index, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=self.out, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def samples(self):
        """Lines written so far."""
        try:
            with open(self.path) as f:
                return sum(1 for line in f if line.count(",") >= 6)
        except (OSError, TypeError):
            return 0

    def stop(self):
        res = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if not self.proc:
            return res
        self.proc.terminate()          # the exact child started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.out.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [s.strip() for s in line.split(",")]
                if len(parts) < 7:
                    continue
                try:
                    sm.append(float(parts[0]))
                    mx.append(float(parts[1]))
                except ValueError:
                    continue
                for nm, v in zip(names, parts[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(nm)
        os.unlink(self.path)
        if sm:
            res = {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                   "samples": len(sm)}
        return res


# ---------------------------------------------------------------------------
# CPU arm
# ---------------------------------------------------------------------------
def cpu_decode_token_seconds(cfg, ctx, reps=1, seed=0, fp32_weights=False):
    """Seconds per decoded token of the CPU path, from a bounded sample: one Mamba-2
    layer, one attention layer, one MoE layer and the lm_head of a single token are
    timed and scaled by the layer counts.  Uses the reference engine's own CPU ops
    (oracle/_ref) on fp16-materialised weights - what its CPU inference path feeds them
    after ops::quant_materialize - when that library exists, else the oracle port.
    fp32_weights: the same ops on fp32 matrices (the engine's unquantised CPU path: nothing
    is dequantised per call).  Returns (seconds per token scaled to the whole model, info);
    info["sample_seconds"] is what one pass over the sample really took."""
    from oracle_lib import OracleOnly, Ref
    ora = OracleOnly()
    use_ref = Ref.available()
    cpu = Ref() if use_ref else ora
    r = np.random.default_rng(seed)
    d = cfg["hidden"]
    q = cfg["qkind"] if cfg["qkind"] >= 0 else 3
    wkind = -2 if fp32_weights else (-1 if use_ref else q)

    def weight(rows, cols):
        w = (r.standard_normal(rows * cols) * 0.02).astype(np.float32)
        if fp32_weights:
            return w
        packed = ora.quantize(w, q)
        return ora.dequantize(packed, rows * cols, q) if use_ref else packed     # fp16 bits or packed

    x = r.standard_normal((1, d)).astype(np.float32)
    times = {}
    # Mamba-2 layer, one token
    nh, dh, ds, k = cfg["mamba_heads"], cfg["mamba_d_head"], cfg["mamba_d_state"], cfg["mamba_d_conv"]
    d_inner = nh * dh
    conv_dim = d_inner + 2 * ds
    proj = d_inner + conv_dim + nh
    margs = (x.reshape(1, 1, d), weight(proj, d), (r.standard_normal((conv_dim, k)) * 0.1).astype(np.float32),
             np.zeros(conv_dim, np.float32), np.zeros(nh, np.float32), np.zeros(nh, np.float32),
             np.ones(nh, np.float32), np.ones(d_inner, np.float32), weight(d, d_inner),
             np.zeros((1, nh, dh, ds), np.float32), 1, 1, d, d_inner, conv_dim, nh, dh, ds, k, 1e-5)

    def best(fn):
        out = []
        for _ in range(max(1, reps)):
            t = time.perf_counter()
            fn()
            out.append(time.perf_counter() - t)
        return min(out)

    times["mamba"] = best(lambda: cpu.mamba2_forward(*margs, wkind))
    # attention layer: 4 projections + decode attention over ctx cached tokens
    H, KV, hd = cfg["n_heads"], cfg["n_kv"], cfg["head_dim"]
    wq, wk, wv, wo = weight(H * hd, d), weight(KV * hd, d), weight(KV * hd, d), weight(d, H * hd)
    kc = r.integers(0, 0x3C00, (ctx, KV * hd)).astype(np.uint16)
    vc = r.integers(0, 0x3C00, (ctx, KV * hd)).astype(np.uint16)

    def attn_layer():
        qv = cpu.linear(x, wq, wkind, 1, d, H * hd)
        cpu.linear(x, wk, wkind, 1, d, KV * hd)
        cpu.linear(x, wv, wkind, 1, d, KV * hd)
        a = cpu.attention_decode_ring(qv.reshape(H, hd), kc, vc, 1, H, KV, hd, 0, 0, ctx, ctx, 0.1, 0)
        cpu.linear(a.reshape(1, -1), wo, wkind, 1, H * hd, d)

    times["attention"] = best(attn_layer)
    # MoE layer
    ne, E, K, SH = cfg["n_experts"], cfg["expert_dim"], cfg["top_k"], cfg["shared_dim"]
    moe = (x, (r.standard_normal((ne, d)) / np.sqrt(d)).astype(np.float32),
           (r.standard_normal(ne) * 0.5 / ne).astype(np.float32), weight(ne * E, d), weight(ne * E, d),
           weight(ne * d, E), weight(SH, d), weight(SH, d), weight(d, SH), d, E, ne, K, SH, wkind)
    times["moe"] = best(lambda: cpu.moe_forward(*moe))
    # lm_head (fp16) on a slice of the vocabulary, scaled
    vs = min(cfg["vocab"], 16384)
    head = r.integers(0, 0x3000, (vs, d)).astype(np.uint16)
    times["lm_head"] = best(lambda: cpu.linear(x, head, -1, 1, d, vs)) * cfg["vocab"] / vs
    n_mamba = sum(1 for t_ in cfg["layer_types"] if t_ == 0)
    n_attn = cfg["n_layers"] - n_mamba
    total = n_mamba * times["mamba"] + n_attn * times["attention"] + cfg["n_layers"] * times["moe"] + times["lm_head"]
    sample = times["mamba"] + times["attention"] + times["moe"] + times["lm_head"] * vs / cfg["vocab"]
    what = ("fp32 weights" if fp32_weights else
            "reference CPU ops on fp16-materialised Q4_K values" if use_ref else "oracle port on packed Q4_K")
    info = {"kind": "reference" if use_ref else "port", "cores": cpu.num_threads(),
            "sample": ("1 Mamba-2 layer + 1 attention layer (ctx %d) + 1 MoE layer + lm_head (%d of %d rows) of one "
                       "decode token, each timed %d time(s) (best kept) and scaled by the layer counts; %s" %
                       (ctx, vs, cfg["vocab"], max(1, reps), what)),
            "sample_seconds": round(sample, 4), "scale_to_full_step": round(total / sample, 2),
            "seconds": {k_: round(v, 4) for k_, v in times.items()}}
    return total, info


def run_reference_arm(args, rank):
    if rank != 0:
        return
    cfg = H_TINY
    # A step of this arm is one pass over the bounded sample (one layer of each kind + a slice
    # of the lm_head); `steps` and `ms_per_step` say what was really timed, `value` is the
    # token rate that sample scales to over the model's 40 layers (cpu_baseline.scale_to_full_step).
    reps = min(max(1, args.steps), 8)
    secs, info = cpu_decode_token_seconds(cfg, args.ctx, reps=reps)
    val = args.batch / secs
    line = {"impl": "reference", "metric": "decode tok/s", "value": val, "unit": "tok/s", "n_gpus": args.gpus,
            "steps": reps, "warmup": 0, "ms_per_step": info["sample_seconds"] * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(cfg, args),
            "sampled": "ms_per_step is one pass over the sample; one full decode step = ms_per_step x "
                       "cpu_baseline.scale_to_full_step, value = batch / that",
            "cpu_baseline": dict(info, value=val, unit="tok/s"),
            "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload_config(cfg, args):
    return {"workload": "Granite-4.0-H-Tiny-shaped model, random-init Q4_K, greedy decode, batch %d, ctx %d" %
                        (args.batch, args.ctx),
            "batch": args.batch, "ctx": args.ctx, "l2": "inputs larger than L2 (>1 GB of weights and state per step)",
            "parallelism": "replicas" if args.gpus > 1 else "single"}


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
def time_kernel_gbs(fn, bytes_per_launch, iters=20):
    """Average duration of one launch with CUDA events on the default stream."""
    import torch
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    return bytes_per_launch / (ms * 1e-3) / 1e9, ms


def peak_bf16_tflops():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f).get("bf16_tflops", 1646.6))
    return 1646.6


def moe_layer_bench(lib, rank, world, tokens=4096, iters=10, graph=False):
    """The MoE layer alone at the H-Tiny shape (hidden 1536, 64 experts, top-6, ffn 512,
    shared 1024, Q4_K) on `tokens` replicated tokens: the single-GPU layer at world 1,
    expert-parallel over NCCL all-to-all at world > 1 (experts sharded, tokens sliced,
    outputs all-gathered).  Device time, max over ranks."""
    import torch
    import torch.distributed as dist
    ep = importlib.import_module(PKG + ".ep")
    d, E, ne, K, SH, q = 1536, 512, 64, 6, 1024, 3
    g = torch.Generator(device="cuda").manual_seed(1234)          # the same weights on every rank

    def packed(n):
        w = torch.randn(n, device="cuda", generator=g) * 0.02
        out = torch.empty(n // 256 * 144, dtype=torch.uint8, device="cuda")
        lib.b200_quantize(w, out, n, q)
        return out

    gates, ups, downs = packed(ne * E * d), packed(ne * E * d), packed(ne * d * E)
    sh = (packed(SH * d), packed(SH * d), packed(d * SH))
    router = torch.randn(ne, d, device="cuda", generator=g) / d ** 0.5
    bias = torch.randn(ne, device="cuda", generator=g) * 0.5 / ne
    x = torch.randn(tokens, d, device="cuda", generator=g)
    layer = ep.ExpertParallelMoE(d, E, ne, K, SH, q, router, bias, ep.shard_experts(gates, ne, rank, world),
                                 ep.shard_experts(ups, ne, rank, world), ep.shard_experts(downs, ne, rank, world), sh)
    out = torch.empty(tokens, d, device="cuda")

    replay = {"fn": None}

    def run(reduce_form=False):
        if world == 1:      # the plain layer call: no exchange, no host read of split sizes
            lib.b200_moe_forward_bias_half(x, router, bias, gates, ups, downs, sh[0], sh[1], sh[2], out, None, None, None,
                                           None, None, None, tokens, d, E, ne, K, SH, q)
        elif reduce_form == "graph":
            replay["fn"](x)
        elif reduce_form:
            layer.forward_reduce(x)
        else:
            layer.forward(x)

    def timed(reduce_form):
        for _ in range(3):
            run(reduce_form)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(iters):
            run(reduce_form)
        t1.record()
        torch.cuda.synchronize()
        t = torch.tensor([t0.elapsed_time(t1) / iters], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    peer = None
    if world > 1:
        # the same layer through the C host over peer memory (include/b200ep.h): no NCCL, no host read
        import ctypes as C
        want = torch.empty(tokens, d, device="cuda")
        want_idx = torch.empty(tokens, K, dtype=torch.int32, device="cuda")
        lib.b200_moe_forward_bias_half(x, router, bias, gates, ups, downs, sh[0], sh[1], sh[2], want, None, want_idx, None,
                                       None, None, None, tokens, d, E, ne, K, SH, q)
        single_ms = time_kernel_gbs(lambda: lib.b200_moe_forward_bias_half(
            x, router, bias, gates, ups, downs, sh[0], sh[1], sh[2], want, None, None, None, None, None, None, tokens, d, E, ne,
            K, SH, q), 1, iters=iters)[1]
        h = C.c_void_p()
        lib.b200_ep_create(C.byref(h), rank, world, d, E, ne, K, SH, q, tokens, 0)
        lib.b200_ep_set_weights(h, router, bias, layer.gates, layer.ups, layer.downs, sh[0], sh[1], sh[2])
        rdv = "/tmp/b200ep_%s_%d" % (os.environ.get("MASTER_PORT", "0"), tokens)
        if rank == 0:
            os.makedirs(rdv, exist_ok=True)
            for f in os.listdir(rdv):
                os.remove(os.path.join(rdv, f))
        dist.barrier()
        lib.b200_ep_rendezvous_dir(h, rdv.encode(), 60000)
        dist.barrier()

        def peer_pass():
            lib.b200_ep_forward(h, x, tokens)

        run_saved = run
        ms_peer = None
        for _ in range(3):
            peer_pass()
        dist.barrier()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(iters):
            peer_pass()
        t1.record()
        torch.cuda.synchronize()
        tt = torch.tensor([t0.elapsed_time(t1) / iters], device="cuda", dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms_peer = float(tt[0])
        po = C.c_void_p()
        lib.b200_ep_output(h, C.byref(po))
        got = torch.empty(tokens, d, device="cuda")
        lib.b200_copy(got, 1, po.value, 1, tokens * d * 4)
        link = C.c_double()
        lib.b200_ep_link_bytes(h, C.byref(link))
        torch.cuda.synchronize()
        diff = (got - want).abs().max()
        same = torch.tensor([float(torch.equal(got, want)), float(lib.raw("b200_stream_status") == 0)], device="cuda",
                            dtype=torch.float64)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        dist.all_reduce(diff, op=dist.ReduceOp.MAX)
        link_t = torch.tensor([link.value], device="cuda", dtype=torch.float64)
        dist.all_reduce(link_t, op=dist.ReduceOp.MAX)
        dist.barrier()
        lib.b200_ep_destroy(h)
        flops_rank = (tokens * K * 3 * 2 * E * d + tokens * 3 * 2 * SH * d) / world
        t_math = flops_rank / (peak_bf16_tflops() * 1e12)
        t_link = float(link_t[0]) / 770e9
        peer = {"ms_per_layer": ms_peer, "single_gpu_ms_per_layer": single_ms, "speedup_vs_single_gpu": single_ms / ms_peer,
                "link_bytes_per_rank": float(link_t[0]),
                "roofline": {"target_ms": max(t_math, t_link) * 1e3, "bound": "tensor" if t_math >= t_link else "nvlink",
                             "math_ms": t_math * 1e3, "link_ms_at_770_GBs": t_link * 1e3,
                             "frac": max(t_math, t_link) * 1e3 / ms_peer},
                "ep_parity": {"bit_identical_to_single_gpu": bool(same[0] == 1.0), "max_abs_diff": float(diff),
                              "status_clean": bool(same[1] == 1.0)},
                "mode": "expert parallel over peer memory: dispatch / return / gather kernels with NVLink stores and epoch flags"}
        del gates, ups, downs, want, got
    ms = timed(False)
    ms_reduce = timed(True) if world > 1 else None
    ms_graph, graph_note = None, None
    if world > 1 and graph:
        try:
            replay["fn"] = layer.graphed_reduce(x)
            ms_graph = timed("graph")
        except Exception as e:                       # capture is an optimisation: report, do not fail the bench
            graph_note = "capture failed: %s" % (str(e).splitlines()[0][:160] if str(e) else type(e).__name__)
    flops = tokens * K * 3 * 2 * E * d + tokens * 3 * 2 * SH * d
    peak_tf = 1646.6
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            peak_tf = float(json.load(f).get("bf16_tflops", peak_tf))
    # every rank computes the shared expert of its own token slice only, so the job's flops are `flops`
    return {"tokens": tokens, "ms_per_layer": ms, "tok_s": tokens / (ms * 1e-3), "tflops": flops / (ms * 1e-3) / 1e12,
            "frac_of_dense_peak": flops / (ms * 1e-3) / 1e12 / (peak_tf * world), "n_gpus": world,
            "mode": "single GPU" if world == 1 else "expert parallel, NCCL all-to-all",
            "ms_per_layer_reduce_form": ms_reduce,
            "ms_per_layer_reduce_form_graph": ms_graph if ms_graph is not None else graph_note,
            "reduce_form": None if ms_reduce is None else "no dispatch: routing per token slice + all-gather of the indices, local experts on the packed rows, one NCCL all-reduce of the output",
            "peer_memory": peer,
            "shape": "hidden 1536, 64 experts, top-6, ffn 512, shared 1024, Q4_K"}


def batch_decode_bench(cfg, batch, ctx, steps, seed):
    """Greedy decode of `batch` sequences at once (per-op mode: every projection and the
    MoE layer run as tensor-core GEMMs over the batch; one CUDA graph per step).  Device
    time only; returns the extra JSON object."""
    import torch
    model = DeviceModel(cfg, batch, ctx + steps + 16, seed=seed)
    model.configure(0, 1)
    g = torch.Generator(device="cuda").manual_seed(7 + seed)
    prompt = torch.randint(0, cfg["vocab"], (batch, ctx), device="cuda", generator=g, dtype=torch.int32)
    tok = torch.empty(batch, dtype=torch.int32, device="cuda")
    model.prefill(prompt, tok)              # untimed: grows the workspaces
    model.reset()
    torch.cuda.synchronize()
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    model.prefill(prompt, tok)
    p1.record()
    for _ in range(3):
        model.step_dev(tok)
    torch.cuda.synchronize()
    prefill_ms = p0.elapsed_time(p1)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        model.step_dev(tok)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    step_bytes = model.step_bytes()
    launches = model.launches()
    model.close()
    peak, _ = peaks()
    return {"batch": batch, "ctx": ctx, "steps": steps, "ms_per_step": ms, "tok_s": batch / (ms * 1e-3),
            "algorithmic_bytes_per_step": step_bytes, "achieved_gbs": step_bytes / (ms * 1e-3) / 1e9,
            "frac_of_hbm_peak": step_bytes / (ms * 1e-3) / 1e9 / peak, "launches_per_step": launches,
            "operands": "fp16 activations x fp16 / in-kernel dequantised Q4_K weights, fp32 accumulation",
            "mode": "per-op, tensor-core GEMM path, CUDA graph",
            "prefill": {"tokens": batch * ctx, "ms": prefill_ms, "tok_s": batch * ctx / (prefill_ms * 1e-3),
                        "note": "%d sequences x %d tokens through b200_decoder_prefill in groups of <= 32768 tokens"
                                % (batch, ctx)}}


def moe_sweep_bench(lib, sizes=(1, 64, 512, 4096)):
    """The MoE layer of the H-Tiny shape at the token counts of the op-level configuration,
    each against the roofline that bounds it: HBM (weights of the experts the tokens touch +
    router + shared expert, read once) for few tokens, dense tensor peak for many."""
    import torch
    d, E, ne, K, SH, q = 1536, 512, 64, 6, 1024, 3
    g = torch.Generator(device="cuda").manual_seed(4321)

    def packed(n):
        w = torch.randn(n, device="cuda", generator=g) * 0.02
        out = torch.empty(n // 256 * 144, dtype=torch.uint8, device="cuda")
        lib.b200_quantize(w, out, n, q)
        return out

    # two weight sets, alternated, so that a size whose weights fit the 126 MB L2 still streams from HBM
    sets = []
    for _ in range(2):
        sets.append(dict(gates=packed(ne * E * d), ups=packed(ne * E * d), downs=packed(ne * d * E),
                         sh=(packed(SH * d), packed(SH * d), packed(d * SH)),
                         router=torch.randn(ne, d, device="cuda", generator=g) / d ** 0.5,
                         bias=torch.randn(ne, device="cuda", generator=g) * 0.5 / ne))    # on the scale of a probability: skewed, ragged loads
    hbm_peak, _ = peaks()
    tf_peak = 1646.6
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            tf_peak = float(json.load(f).get("bf16_tflops", tf_peak))
    out = []
    for T in sizes:
        x = torch.randn(T, d, device="cuda", generator=g)
        y = torch.empty(T, d, device="cuda")
        idx = torch.empty(T, K, dtype=torch.int32, device="cuda")
        state = {"i": 0}

        def run():
            w = sets[state["i"] & 1]
            state["i"] += 1
            lib.b200_moe_forward_bias_half(x, w["router"], w["bias"], w["gates"], w["ups"], w["downs"], w["sh"][0],
                                           w["sh"][1], w["sh"][2], y, None, idx, None, None, None, None, T, d, E, ne, K,
                                           SH, q)

        _, ms = time_kernel_gbs(run, 0, iters=20)
        touched = int(torch.unique(idx).numel())
        wbytes = (touched * 3 * E * d + 3 * SH * d) // 256 * 144 + ne * d * 4
        flops = T * K * 3 * 2 * E * d + T * 3 * 2 * SH * d
        gbs, tfs = wbytes / (ms * 1e-3) / 1e9, flops / (ms * 1e-3) / 1e12
        bound = "hbm" if wbytes / (hbm_peak * 1e9) > flops / (tf_peak * 1e12) else "tensor"
        out.append({"tokens": T, "ms_per_layer": ms, "experts_touched": touched, "weight_bytes": wbytes,
                    "achieved_gbs": gbs, "frac_of_hbm_peak": gbs / hbm_peak, "tflops": tfs,
                    "frac_of_dense_peak": tfs / tf_peak, "bound": bound,
                    "operands": "fp32 (exact dequantised weights; the shared expert as an fp16 tensor-core GEMM from 9 tokens on)"
                                if T * K <= 12 * ne else "fp16 x in-kernel dequantised Q4_K, fp32 accumulation"})
    return out


def mamba_ops_bench(lib):
    """Mamba-2 at the op level (the shapes of the op-level configuration): b200_mamba2_forward_half
    over [8, 4096] tokens with 48 heads x 64 and d_state 128 - causal conv, chunked SSD scan,
    gated norm at the full inner width of 3072; the projections in front and behind run at a
    model width of 256 so that they stay a small part (their time is inside the figure) - and
    the single-token state update for 64 sequences (b200_mamba2_step_batched)."""
    import torch
    B, T, d, nh, dh, ds, k, q = 8, 4096, 256, 48, 64, 128, 4, 3
    d_inner, conv_dim = nh * dh, nh * dh + 2 * ds
    proj = d_inner + conv_dim + nh
    g = torch.Generator(device="cuda").manual_seed(99)

    def packed(n, std):
        w = torch.randn(n, device="cuda", generator=g) * std
        o = torch.empty(n // 256 * 144, dtype=torch.uint8, device="cuda")
        lib.b200_quantize(w, o, n, q)
        return o

    w_in, w_out = packed(proj * d, 0.05), packed(d * d_inner, 0.02)
    conv_w = torch.randn(conv_dim * k, device="cuda", generator=g) * 0.1
    conv_b = torch.zeros(conv_dim, device="cuda")
    dt_bias = torch.log(torch.expm1(torch.rand(nh, device="cuda", generator=g) * (1e-1 - 1e-3) + 1e-3))
    a_log = torch.rand(nh, device="cuda", generator=g) * float(np.log(16.0))
    D = torch.randn(nh, device="cuda", generator=g)
    norm_w = torch.ones(d_inner, device="cuda")
    x = torch.randn(B * T * d, device="cuda", generator=g)
    state = torch.zeros(B * nh * dh * ds, device="cuda")
    out = torch.empty(B * T * d, device="cuda")

    def fwd():
        lib.b200_mamba2_forward_half(x, w_in, conv_w, conv_b, dt_bias, a_log, D, norm_w, w_out, state, out, B, T, d,
                                     d_inner, conv_dim, nh, dh, ds, k, 1e-5, q)

    # algorithmic traffic of the scan itself: x and y [B,T,d_inner] bf16-sized in the op-level
    # description; here the post-projection tensors are fp32: x, B, C, dt in, y out, state in + out
    scan_bytes = B * T * (d_inner * 4 + 2 * ds * 4 + nh * 4 + d_inner * 4) + 2 * B * nh * dh * ds * 4
    config_bytes = 451e6          # the same tensors with x and y in bf16, as the op-level configuration states them
    scan_flops = B * nh * (T // 128) * 2 * 128 * (128 * ds + 128 * dh + 2 * ds * dh)
    gbs, ms = time_kernel_gbs(fwd, scan_bytes, iters=5)
    peak, _ = peaks()
    res = {"ssd_prefill": {"shape": "[8, 4096, 48, 64], d_state 128, chunk 128, Q4_K projections at width 256 included",
                           "ms": ms, "tok_s": B * T / (ms * 1e-3), "algorithmic_bytes": scan_bytes,
                           "algorithmic_bytes_bf16_boundary": config_bytes,
                           "achieved_gbs": gbs, "frac_of_hbm_peak": gbs / peak,
                           "scan_tflops": scan_flops / (ms * 1e-3) / 1e12,
                           "operands": "fp16 per-head operands, fp32 dt / decays / carry / accumulation"}}
    # batch-64 single-token update: state read + written
    Bs = 64
    xs = torch.randn(Bs * d, device="cuda", generator=g)
    conv_state = torch.zeros(Bs * conv_dim * (k - 1), device="cuda")
    # several state sets, alternated: 64 sequences are 100 MB, below the L2 size
    states = [torch.zeros(Bs * nh * dh * ds, device="cuda") for _ in range(3)]
    outs = torch.empty(Bs * d, device="cuda")
    it = {"i": 0}

    def step():
        st = states[it["i"] % 3]
        it["i"] += 1
        lib.b200_mamba2_step_batched(xs, w_in, conv_w, conv_b, dt_bias, a_log, D, norm_w, w_out, conv_state, st, outs, Bs,
                                     d, d_inner, conv_dim, nh, dh, ds, k, 1e-5, q)

    step_bytes = 2 * Bs * nh * dh * ds * 4
    gbs2, ms2 = time_kernel_gbs(step, step_bytes, iters=30)
    res["state_update_b64"] = {"shape": "64 sequences x [48, 64, 128] fp32 state", "ms": ms2,
                               "algorithmic_bytes": step_bytes, "achieved_gbs": gbs2, "frac_of_hbm_peak": gbs2 / peak,
                               "operands": "fp32"}
    return res


def quantize_bench(lib):
    """The load-time quantisers on one H-Tiny expert tensor (64 x 512 x 1536 fp32 = 201 MB in, larger than
    L2): fp32 read + packed bytes written per second, per storage kind."""
    import torch
    n = 64 * 512 * 1536
    x = torch.randn(n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(5)) * 0.02
    peak, _ = peaks()
    out = {}
    for kind, name, be, bb in ((2, "q8_0", 32, 34), (0, "q4_0", 32, 18), (4, "q4_0_gguf_rule", 32, 18), (1, "q4_1", 32, 20),
                               (3, "q4_k", 256, 144)):
        dst = torch.empty(n // be * bb, dtype=torch.uint8, device="cuda")
        nbytes = n * 4 + dst.numel()
        gbs, ms = time_kernel_gbs(lambda: lib.b200_quantize(x, dst, n, kind), nbytes, iters=10)
        out[name] = {"ms": ms, "achieved_gbs": gbs, "frac_of_hbm_peak": gbs / peak, "weights_per_s": n / (ms * 1e-3)}
    return out


def config1_bench():
    """Config 1 end to end: the 8-layer hybrid (hidden 768, vocabulary 32768, Q8_0), a 128-token prompt
    through b200_decoder_prefill, then 128 greedy steps through b200_decoder_step_host (host token in,
    host pick out, a synchronise per token) - wall clock around the whole generation."""
    import torch
    from model_util import CONFIG_1
    cfg = dict(CONFIG_1)
    model = DeviceModel(cfg, 1, 128 + 128 + 16, seed=0)
    model.configure(1, 1)
    prompt = torch.randint(0, cfg["vocab"], (1, 128), device="cuda", dtype=torch.int32,
                           generator=torch.Generator(device="cuda").manual_seed(1))
    tok = torch.empty(1, dtype=torch.int32, device="cuda")
    tin, tout = np.zeros(1, np.int32), np.zeros(1, np.int32)

    def generate():
        model.reset()
        model.prefill(prompt, tok)
        tin[0] = int(tok.cpu()[0])
        for _ in range(128):
            model.step_host(tin, tout)
            tin[0] = tout[0]

    generate()                      # sizes workspaces, records the graph
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    generate()
    torch.cuda.synchronize()
    sec = time.perf_counter() - t0
    model.close()
    return {"workload": "8 layers (6 Mamba-2 + 2 GQA), hidden 768, vocabulary 32768, Q8_0, batch 1: 128-token prompt + 128 greedy steps",
            "seconds": sec, "decode_tok_s_incl_prompt": 128 / sec, "ms_per_generated_token": sec / 128 * 1e3,
            "mode": "prefill through the many-token kernels, steps through b200_decoder_step_host (fused mode, CUDA graph)"}


def config5_bench(steps=256, n_seq=64, lo=256, hi=8192):
    """The ragged serving workload on one GPU: the H-Small-shaped model (hidden 4096, 36 Mamba-2 + 4 GQA
    layers, 72 experts / top-10, Q4_K, random-init), 64 sequences with prompt lengths uniform in
    [256, 8192] (seed 7) through b200_decoder_prefill_ragged, then `steps` greedy decode steps of all 64
    sequences at their own positions (paged KV, page 64).  The 8-GPU expert-parallel form of this
    model's MoE layer is measured separately (the moe blocks under --gpus N)."""
    import torch
    cfg = H_SMALL
    lengths = np.random.default_rng(7).integers(lo, hi + 1, n_seq).astype(np.int32)
    total = int(lengths.sum())
    t0 = time.time()
    model = DeviceModel(cfg, n_seq, int(lengths.max()) + steps + 16, seed=5)
    model.configure(0, 1)
    build_s = time.time() - t0
    g = torch.Generator(device="cuda").manual_seed(8)
    prompt = torch.randint(0, cfg["vocab"], (total,), device="cuda", generator=g, dtype=torch.int32)
    tok = torch.empty(n_seq, dtype=torch.int32, device="cuda")
    lib = model.lib
    lib.b200_decoder_prefill_ragged(model.handle, prompt, lengths.ctypes.data, tok)      # untimed: sizes the workspaces
    model.reset()
    torch.cuda.synchronize()
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    lib.b200_decoder_prefill_ragged(model.handle, prompt, lengths.ctypes.data, tok)
    p1.record()
    for _ in range(3):
        model.step_dev(tok)
    torch.cuda.synchronize()
    prefill_ms = p0.elapsed_time(p1)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        model.step_dev(tok)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    status = lib.raw("b200_stream_status")
    weights = sum(t.numel() * t.element_size() for t in model.tensors.values())
    free, total_mem = torch.cuda.mem_get_info()
    peak, _ = peaks()
    # per step: every weight matrix once (64 sequences x 10 experts touch all 72 experts), Mamba state read + written,
    # the KV of every sequence at its own length
    d_inner = cfg["mamba_heads"] * cfg["mamba_d_head"]
    state = 2 * n_seq * 36 * d_inner * cfg["mamba_d_state"] * 4
    kv = float((lengths.astype(np.int64) + 3 + steps // 2).sum()) * 4 * 2 * cfg["n_kv"] * cfg["head_dim"] * 2
    step_bytes = weights - cfg["vocab"] * cfg["hidden"] * 2 * 0 + state + kv
    out = {"model": "Granite-4.0-H-Small-shaped, random-init Q4_K, %.1f GB of weights" % (weights / 1e9),
           "sequences": n_seq, "prompt_lengths": "uniform [%d, %d], seed 7: min %d, max %d, %d tokens in all" % (
               lo, hi, int(lengths.min()), int(lengths.max()), total),
           "prefill_ms": prefill_ms, "prefill_tok_s": total / (prefill_ms * 1e-3),
           "decode_steps": steps, "ms_per_step": ms, "decode_tok_s": n_seq / (ms * 1e-3),
           "algorithmic_bytes_per_step": step_bytes, "achieved_gbs": step_bytes / (ms * 1e-3) / 1e9,
           "frac_of_hbm_peak": step_bytes / (ms * 1e-3) / 1e9 / peak,
           "device_memory_used_gb": (total_mem - free) / 1e9, "model_build_s": build_s, "status_clean": status == 0,
           "mode": "ragged prefill in groups of <= 32768 tokens; per-op batched decode, tensor-core GEMM path, one CUDA graph per step"}
    model.close()
    return out


def gemm_only_bench():
    """The many-token kernels alone: fp16 and Q4_K linears of the in_proj shape at 4096 rows,
    and the MoE layer at 512 and 4096 tokens.  One JSON line; ~1 GB on the device."""
    import torch
    lib = importlib.import_module(PKG).lib()
    M, K, N = 4096, 1536, 6448
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(M, K, device="cuda", generator=g)
    w16 = (torch.randn(N, K, device="cuda", generator=g) * 0.02).half()
    wq = torch.empty(N * K // 256 * 144, dtype=torch.uint8, device="cuda")
    lib.b200_quantize(w16.float().reshape(-1).contiguous(), wq, N * K, 3)
    y = torch.empty(M, N, device="cuda")
    flops = 2.0 * M * K * N

    def timed(fn, iters=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    ms16 = timed(lambda: lib.b200_linear_forward_fp16(x, w16, y, M, K, N))
    msq = timed(lambda: lib.b200_linear_forward_q4(x, wq, y, M, K, N, 3))
    out = {"linear_fp16": {"M": M, "K": K, "N": N, "ms": ms16, "tflops": flops / ms16 / 1e9},
           "linear_q4k": {"M": M, "K": K, "N": N, "ms": msq, "tflops": flops / msq / 1e9},
           "moe_512": moe_layer_bench(lib, 0, 1, tokens=512), "moe_4096": moe_layer_bench(lib, 0, 1, tokens=4096),
           "moe_16384": moe_layer_bench(lib, 0, 1, tokens=16384)}
    if lib.raw("b200_stream_status") != 0:
        raise RuntimeError(lib.last_error())
    print(json.dumps(out))


def prefill_only_bench(args):
    """The prompt path alone: `--ctx` tokens per sequence, `--batch` sequences."""
    import torch
    cfg = dict(H_TINY)
    if args.small:
        cfg.update(n_layers=4, layer_types=[0, 1, 0, 0], vocab=8192)
    model = DeviceModel(cfg, args.batch, args.ctx + 8, seed=0)
    g = torch.Generator(device="cuda").manual_seed(1)
    prompt = torch.randint(0, cfg["vocab"], (args.batch, args.ctx), device="cuda", generator=g, dtype=torch.int32)
    tok = torch.empty(args.batch, dtype=torch.int32, device="cuda")
    model.prefill(prompt, tok)
    times = []
    for _ in range(3):
        model.reset()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        model.prefill(prompt, tok)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    if model.lib.raw("b200_stream_status") != 0:
        raise RuntimeError(model.lib.last_error())
    n = args.batch * args.ctx
    ms = min(times)
    print(json.dumps({"prefill": {"batch": args.batch, "tokens_per_sequence": args.ctx, "layers": cfg["n_layers"],
                                  "ms": ms, "tok_s": n / (ms * 1e-3)}}))
    model.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--ctx", type=int, default=4096, help="tokens in the KV cache / state before the timed steps")
    ap.add_argument("--fused", type=int, default=1)
    ap.add_argument("--graph", type=int, default=1)
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--small", action="store_true", help="4-layer model (development only; not a bench number)")
    ap.add_argument("--quick", action="store_true", help="skip the op-level and batch-64 blocks")
    ap.add_argument("--ep-graph", action="store_true",
                    help="N > 1: also time the dispatch-free expert-parallel layer replayed as one CUDA graph "
                         "(NCCL all-reduce captured with it)")
    ap.add_argument("--profile-step", action="store_true",
                    help="after the timed steps run ONE more step between cudaProfilerStart/Stop and exit "
                         "(for ncu --profile-from-start off: DRAM bytes of every launch of a step)")
    ap.add_argument("--only", default="", choices=["", "gemm", "prefill", "config5", "moe64", "quantize"],
                    help="gemm: time the tensor-core linears and the MoE layer alone (small; also the profiling case); "
                         "prefill: time the prompt path alone (with --small: the profiling case); "
                         "config5: the H-Small-shaped model on the ragged 64-sequence workload (about 40 GB on the device); "
                         "moe64 / quantize: the MoE layer on 64 tokens / the load-time quantisers alone (profiling cases)")
    args = ap.parse_args()
    if args.only == "gemm":
        gemm_only_bench()
        return
    if args.only == "prefill":
        prefill_only_bench(args)
        return
    if args.only == "moe64":
        # the MoE layer on a decode batch of 64 tokens (small profiling case)
        lib = importlib.import_module(PKG).lib()
        print(json.dumps({"moe_sweep": moe_sweep_bench(lib, sizes=(64,))}))
        return
    if args.only == "quantize":
        lib = importlib.import_module(PKG).lib()
        print(json.dumps({"quantizers": quantize_bench(lib)}))
        return
    if args.only == "config5":
        print(json.dumps({"config5": config5_bench(steps=args.steps if args.steps != 128 else 256)}))
        return

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    cfg = dict(H_TINY)
    if args.small:
        cfg.update(n_layers=4, layer_types=[0, 1, 0, 0], vocab=8192)
    B = args.batch
    W = max(3, args.warmup)
    total_ctx = args.ctx + W + 2 * args.steps + 8 + 1600     # + room for the clock sampler's extension
    model = DeviceModel(cfg, B, total_ctx, seed=rank)
    lib = model.lib
    model.configure(args.fused, args.graph)

    # prompt: ctx uniform token ids per sequence through the prompt path (once untimed: it
    # grows the workspaces; then timed from empty sequences)
    g = torch.Generator(device="cuda").manual_seed(1 + rank)
    prompt = torch.randint(0, cfg["vocab"], (B, max(args.ctx, 1)), device="cuda", generator=g, dtype=torch.int32)
    tok = torch.empty(B, dtype=torch.int32, device="cuda")
    prefill_ms = None
    if args.ctx >= 1:
        model.prefill(prompt, tok)
        model.reset()
        torch.cuda.synchronize()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record()
        model.prefill(prompt, tok)
        p1.record()
        torch.cuda.synchronize()
        prefill_ms = p0.elapsed_time(p1)
    else:
        tok.copy_(prompt[:, 0])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing -------------------------------------------------
    for _ in range(W):
        model.step_dev(tok)
    barrier()
    launches_before = lib.b200_kernel_launches()
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        model.step_dev(tok)
    e1.record()
    barrier()
    ms_dev = e0.elapsed_time(e1)
    step_bytes = model.step_bytes()
    launches_per_step = model.launches()

    # ---- end to end through host buffers -----------------------------------------
    tok_h = tok.cpu().numpy().copy()
    out_h = np.empty(B, np.int32)
    for _ in range(3):
        model.step_host(tok_h, out_h)
        tok_h[:] = out_h
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        model.step_host(tok_h, out_h)
        tok_h[:] = out_h
    torch.cuda.synchronize()
    sec_e2e = time.perf_counter() - t0
    # a short run can end before nvidia-smi has written its first line: keep the same load
    # on the GPU (untimed) until two samples exist, for at most three seconds
    extended = False
    t_end, rounds = time.time() + 3.0, 0
    while sampler.proc and sampler.samples() < 2 and time.time() < t_end and rounds < 96:
        extended = True
        rounds += 1
        for _ in range(16):
            model.step_dev(tok)
        torch.cuda.synchronize()
    clocks = sampler.stop()
    clocks["window"] = "timed region, then the same decode load until two samples existed" if extended else "timed region"

    if args.profile_step:
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        model.step_dev(tok)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(json.dumps({"profiled_step": {"ms_per_step_before": ms_dev / args.steps, "launches": launches_per_step,
                                            "algorithmic_bytes": step_bytes}}))
        model.close()
        return

    times = torch.tensor([ms_dev, sec_e2e * 1e3], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_dev, ms_e2e = float(times[0]), float(times[1])

    # ---- dominant kernel: the lm_head GEMV (fp16 [vocab, hidden], the largest single read)
    peak, peak_src = peaks()
    V, d = cfg["vocab"], cfg["hidden"]
    xb = torch.randn(B, d, device="cuda")
    logits = torch.empty(B, V, device="cuda")
    head = model.tensors[(-1, "embed")]
    head_bytes = V * d * 2
    head_gbs, head_ms = time_kernel_gbs(lambda: lib.b200_linear_forward_fp16(xb, head, logits, B, d, V), head_bytes)
    # and the Q4_K projection kernel on one layer's in_proj (alternating layers so L2 holds nothing)
    mamba_layers = [l for l, t in enumerate(cfg["layer_types"]) if t == 0]
    proj_n = 2 * cfg["mamba_heads"] * cfg["mamba_d_head"] + 2 * cfg["mamba_d_state"] + cfg["mamba_heads"]
    yproj = torch.empty(B, proj_n, device="cuda")
    state = {"i": 0}

    def q4k_call():
        l = mamba_layers[state["i"] % len(mamba_layers)]
        state["i"] += 1
        lib.b200_linear_forward_q4(xb, model.tensors[(l, "w_in")], yproj, B, d, proj_n, cfg["qkind"])

    q4k_bytes = proj_n * d // 256 * 144
    q4k_gbs, q4k_ms = time_kernel_gbs(q4k_call, q4k_bytes, iters=len(mamba_layers) * 2)
    moe = moe_layer_bench(lib, rank, world, graph=args.ep_graph)
    ep_sweep = None
    if world > 1 and not args.quick:
        # where the exchange pays: more tokens per pass (the prompt side of the workload)
        ep_sweep = [moe_layer_bench(lib, rank, world, tokens=t, iters=5) for t in (16384, 65536)]
    batch64 = moe_sweep = mamba_ops = quantizers = config1 = None
    if world == 1 and B == 1 and not args.small and not args.quick:
        model.close()
        model = None
        moe_sweep = moe_sweep_bench(lib)
        mamba_ops = mamba_ops_bench(lib)
        quantizers = quantize_bench(lib)
        config1 = config1_bench()
        batch64 = batch_decode_bench(cfg, 64, 4096, 16, seed=rank)

    default_workload = (B == 1 and args.ctx == 4096 and args.fused == 1 and args.graph == 1 and not args.small)
    step_traffic = measured_step_traffic(launches_per_step) if default_workload else None
    if rank == 0:
        tok_s = B * args.steps * world / (ms_dev * 1e-3)
        e2e_tok_s = B * args.steps * world / (ms_e2e * 1e-3)
        step_gbs = step_bytes / (ms_dev / args.steps * 1e-3) / 1e9
        line = {
            "metric": "decode tok/s", "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": W, "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(cfg, args),
            "dtype_note": "the decode step computes in fp32 on exact dequantised weights (activations enter the "
                          "dot products as fp16 head + tail pairs, 22 bits); every many-token block states its own operands",
            "e2e": {"value": e2e_tok_s, "unit": "tok/s", "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B,
                    "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
            # the whole step is one CUDA graph of weight-streaming kernels, none of which
            # holds a majority of the time: the step itself is the unit whose bytes / time
            # is compared with the copy bandwidth; its two extremes follow as separate keys
            "roofline": {"bound": "hbm", "achieved": step_gbs, "peak": peak, "unit": "GB/s",
                         "frac": step_gbs / peak, "traffic": step_traffic, "peak_source": peak_src,
                         "kernel": "decode step (%d launches in one CUDA graph)" % launches_per_step,
                         "ms_per_launch": ms_dev / args.steps, "algorithmic_bytes_per_launch": step_bytes,
                         "fused": args.fused, "graph": args.graph},
            "roofline_lm_head": {"bound": "hbm", "achieved": head_gbs, "peak": peak, "unit": "GB/s",
                                 "frac": head_gbs / peak, "kernel": "streamed fp16 GEMV (lm_head [%d,%d])" % (V, d),
                                 "ms_per_launch": head_ms, "algorithmic_bytes_per_launch": head_bytes},
            "roofline_q4k_gemv": {"bound": "hbm", "achieved": q4k_gbs, "peak": peak, "unit": "GB/s",
                                  "frac": q4k_gbs / peak, "kernel": "streamed Q4_K GEMV (in_proj [%d,%d])" % (proj_n, d),
                                  "ms_per_launch": q4k_ms, "algorithmic_bytes_per_launch": q4k_bytes},
            "moe_layer": moe,
            "moe_sweep": moe_sweep,
            "mamba_ops": mamba_ops,
            "quantizers": quantizers,
            "config1": config1,
            "moe_layer_ep_sweep": ep_sweep,
            "batch64": batch64,
            "prefill": None if prefill_ms is None else {
                "tokens": B * args.ctx, "ms": prefill_ms, "tok_s": B * args.ctx / (prefill_ms * 1e-3),
                "operands": "fp16 activations x fp16 / in-kernel dequantised Q4_K weights, fp32 accumulation",
                "mode": "b200_decoder_prefill: tensor-core GEMMs, chunked SSD scan, tensor-core attention, grouped MoE"},
        }
        if not args.no_cpu and world == 1:
            secs, info = cpu_decode_token_seconds(cfg, args.ctx, reps=8)
            line["cpu_baseline"] = dict(info, value=B / secs, unit="tok/s")
            secs32, info32 = cpu_decode_token_seconds(cfg, args.ctx, reps=4, fp32_weights=True)
            line["cpu_baseline_fp32"] = dict(info32, value=B / secs32, unit="tok/s")
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line))
    if model is not None:
        model.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
