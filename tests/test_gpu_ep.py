"""GPU parity: the expert-parallel building blocks of the C ABI.

One GPU is enough: world_size 1 runs jdm-ghassan_v1_flach_b200/ep.py end to end on the
device, and G virtual ranks are emulated in one process by carrying the rows between
the per-rank steps with tensor copies where the ranks would use all-to-all - the
device code (routing of a slice, packing, experts on (source, expert) blocks through
the group map, combine) is exactly what a rank runs."""
import importlib

import numpy as np
import pytest
import torch

from cases import moe_case

pytestmark = pytest.mark.gpu

ep = importlib.import_module("jdm-ghassan_v1_flach_b200.ep")


def _dev_case(oracle, seed, T, d, E, ne, K, SH, wkind):
    from gpu_util import dev
    c = moe_case(oracle, seed, T, d, E, ne, K, SH, wkind)
    return c, {k: dev(v) for k, v in c.items()}


def _single_gpu_layer(dc, T, d, E, ne, K, SH, wkind):
    from gpu_util import empty, host, ops
    out, idx = empty((T, d)), empty((T, K), torch.int32)
    ops.moe_forward_bias_half(dc["x"], dc["router_w"], dc["router_bias"], dc["gates"], dc["ups"], dc["downs"], dc["sh_g"],
                              dc["sh_u"], dc["sh_d"], out, None, idx, None, None, None, None, T, d, E, ne, K, SH, wkind)
    return host(out), host(idx)


@pytest.mark.parametrize("wkind,d,E,SH", [(3, 256, 256, 512), (-1, 128, 64, 64), (2, 256, 256, 256)])
def test_world_size_one_equals_the_layer(oracle, wkind, d, E, SH):
    from gpu_util import host
    T, ne, K = 200, 16, 2            # more than 12 rows per expert: the single GPU takes the tensor-core path too
    c, dc = _dev_case(oracle, 7, T, d, E, ne, K, SH, wkind)
    layer = ep.ExpertParallelMoE(d, E, ne, K, SH, wkind, dc["router_w"], dc["router_bias"], dc["gates"], dc["ups"],
                                 dc["downs"], (dc["sh_g"], dc["sh_u"], dc["sh_d"]))
    out, idx = layer.forward(dc["x"])
    want, want_idx = _single_gpu_layer(dc, T, d, E, ne, K, SH, wkind)
    assert np.array_equal(host(idx), want_idx)
    # same kernels, same order of additions: identical bits
    assert np.array_equal(host(out).view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("G", [2, 4, 8])
def test_virtual_ranks_equal_the_layer(oracle, G):
    """Config-3 shape (hidden 1536, 64 experts, top-6, Q4_K) on 200 tokens, G ranks emulated."""
    from gpu_util import fp16_close, host
    T, d, E, ne, K, SH, wkind = 200, 1536, 512, 64, 6, 1024, 3
    c, dc = _dev_case(oracle, 11, T, d, E, ne, K, SH, wkind)
    be = ep.CudaBackend()
    nl = ne // G
    shards = [tuple(ep.shard_experts(dc[k], ne, r, G) for k in ("gates", "ups", "downs")) for r in range(G)]
    # phase 1 on every rank: route + pack its slice
    st = []
    for r in range(G):
        lo, hi = ep.token_slice(T, r, G)
        xs = dc["x"][lo:hi].contiguous()
        idx, w = be.route(xs, dc["router_w"], dc["router_bias"], ne, K)
        rows, inv, offsets = be.dispatch_pack(xs, idx, ne)
        counts = (offsets[1:] - offsets[:-1]).view(G, nl)
        st.append(dict(xs=xs, idx=idx, w=w, rows=rows, inv=inv, offsets=offsets, counts=counts))
    # "all-to-all": destination q receives from every source r its block of rows
    outs = [None] * G
    y_back = [[None] * G for _ in range(G)]          # [source][dest] results travelling home
    for q in range(G):
        blocks, cnts = [], []
        for r in range(G):
            o = st[r]["offsets"]
            lo, hi = int(o[q * nl]), int(o[(q + 1) * nl])
            blocks.append(st[r]["rows"][lo:hi])
            cnts.append(st[r]["counts"][q])
        got = torch.cat(blocks, 0)
        recv_counts = torch.cat(cnts).to(torch.int32)
        goff = torch.zeros(G * nl + 1, dtype=torch.int32, device="cuda")
        goff[1:] = torch.cumsum(recv_counts, 0)
        gmap = torch.arange(nl, dtype=torch.int32, device="cuda").repeat(G)
        y = be.experts_rows(got, goff, gmap, *shards[q], nl, d, E, wkind)
        pos = 0
        for r in range(G):
            n = int(cnts[r].sum())
            y_back[r][q] = y[pos:pos + n]
            pos += n
    sh = (dc["sh_g"], dc["sh_u"], dc["sh_d"])
    for r in range(G):
        y = torch.cat(y_back[r], 0)
        outs[r] = be.shared_combine(st[r]["xs"], sh, y, st[r]["inv"], st[r]["w"], K, SH, wkind)
    out = host(torch.cat(outs, 0))
    idx = host(torch.cat([s["idx"] for s in st], 0))
    want, want_idx = _single_gpu_layer(dc, T, d, E, ne, K, SH, wkind)
    assert np.array_equal(idx, want_idx)                          # routing identical to the 1-GPU run
    # every row is the same dot products in the same order, whichever tile it sat in
    assert np.array_equal(out.view(np.uint32), want.view(np.uint32))
    # and the layer itself against the CPU oracle on a sample of tokens
    sample = np.array([0, 1, 99, 100, 199])
    sub = dict(c, x=np.ascontiguousarray(c["x"][sample]))
    ref, _, _, _ = oracle.moe_forward(sub["x"], c["router_w"], c["router_bias"], c["gates"], c["ups"], c["downs"],
                                      c["sh_g"], c["sh_u"], c["sh_d"], d, E, ne, K, SH, wkind)
    fp16_close(out[sample], ref)


@pytest.mark.parametrize("G", [2, 8])
def test_dispatch_free_form_with_virtual_ranks(oracle, G):
    """forward_reduce(): every virtual rank routes all tokens, runs its own experts and forms
    a partial output; the sum of the partials (what the all-reduce computes) is the layer.
    The K expert outputs of a token are added per rank first, so the comparison with the
    single-GPU layer is to summation order, not bit for bit.  Two rounds: the second one
    reuses each rank's persistent row buffer with different tokens."""
    from gpu_util import SUM_ORDER, host
    T, d, E, ne, K, SH, wkind = 200, 1536, 512, 64, 6, 1024, 3
    layers = None
    for seed in (11, 12):
        c, dc = _dev_case(oracle, seed, T, d, E, ne, K, SH, wkind)
        if layers is None:
            weights = dc
            layers = []
            for r in range(G):
                sh = tuple(ep.shard_experts(dc[k], ne, r, G) for k in ("gates", "ups", "downs"))
                layer = ep.ExpertParallelMoE(d, E, ne, K, SH, wkind, dc["router_w"], dc["router_bias"], *sh,
                                             (dc["sh_g"], dc["sh_u"], dc["sh_d"]))
                layer.rank, layer.world, layer.n_local = r, G, ne // G
                layer._reduce = lambda t: t                       # the test adds the partials itself
                layers.append(layer)
        x = dc["x"]
        total, idx0 = None, None
        for layer in layers:
            part, idx = layer.forward_reduce(x)
            total = part.clone() if total is None else total + part
            idx0 = idx if idx0 is None else idx0
            assert torch.equal(idx, idx0)                           # the same routing on every rank
        wd = dict(weights, x=x)
        want, want_idx = _single_gpu_layer(wd, T, d, E, ne, K, SH, wkind)
        assert np.array_equal(host(idx0), want_idx)
        np.testing.assert_allclose(host(total), want, **SUM_ORDER)


def test_dispatch_free_form_few_rows_leaves_other_ranks_rows_alone(oracle):
    """Few tokens and few local experts: the shape at which a plain GEMM cuts K across CTAs
    and adds the partial sums in a second pass over all rows.  The grouped GEMM of a rank
    covers only its own experts' rows, so that pass must not run there: the rows of other
    ranks' experts keep the persistent buffer's (finite) contents.  The split-K workspace is
    filled with NaN first by a plain linear on NaN activations."""
    from gpu_util import SUM_ORDER, dev, empty, host, ops
    T, d, E, ne, K, SH, wkind, G = 48, 1024, 256, 8, 2, 256, 3, 4
    c, dc = _dev_case(oracle, 31, T, d, E, ne, K, SH, wkind)
    # a plain linear of the same few rows takes the split-K path: poison its workspace
    r = np.random.default_rng(5)
    w = dev(oracle.quantize((r.standard_normal(512 * d) * 0.02).astype(np.float32), 3))
    nan_x = torch.full((T * K, d), float("nan"), device="cuda")
    ops.linear_forward_q4(nan_x, w, empty((T * K, 512)), T * K, d, 512, 3)
    total, idx0 = None, None
    for rank in range(G):
        sh = tuple(ep.shard_experts(dc[k], ne, rank, G) for k in ("gates", "ups", "downs"))
        layer = ep.ExpertParallelMoE(d, E, ne, K, SH, wkind, dc["router_w"], dc["router_bias"], *sh,
                                     (dc["sh_g"], dc["sh_u"], dc["sh_d"]))
        layer.rank, layer.world, layer.n_local = rank, G, ne // G
        layer._reduce = lambda t: t
        part, idx = layer.forward_reduce(dc["x"])
        assert torch.isfinite(part).all()
        total = part.clone() if total is None else total + part
        idx0 = idx
    want, want_idx = _single_gpu_layer(dc, T, d, E, ne, K, SH, wkind)
    assert np.array_equal(host(idx0), want_idx)
    # (at this size the single-GPU layer runs its fp32 decode-batch kernels, the ranks the
    # tensor-core GEMM on fp16 operands: compared at the fp16 bound)
    from gpu_util import fp16_close
    fp16_close(host(total), want)


def test_dispatch_free_form_replays_as_a_cuda_graph(oracle):
    """graphed_reduce(): the captured layer gives the same bits as the eager call, also for a
    second input of the same shape."""
    from gpu_util import host, pkg
    T, d, E, ne, K, SH, wkind = 128, 256, 256, 16, 2, 512, 3
    c, dc = _dev_case(oracle, 21, T, d, E, ne, K, SH, wkind)
    layer = ep.ExpertParallelMoE(d, E, ne, K, SH, wkind, dc["router_w"], dc["router_bias"], dc["gates"], dc["ups"],
                                 dc["downs"], (dc["sh_g"], dc["sh_u"], dc["sh_d"]))
    replay = layer.graphed_reduce(dc["x"])
    for seed in (21, 22):
        x = _dev_case(oracle, seed, T, d, E, ne, K, SH, wkind)[1]["x"]
        want, want_idx = layer.forward_reduce(x)
        torch.cuda.synchronize()
        got, got_idx = replay(x)
        torch.cuda.synchronize()
        assert torch.equal(got_idx, want_idx)
        assert np.array_equal(host(got).view(np.uint32), host(want).view(np.uint32))
    assert pkg.lib().raw("b200_stream_status") == 0


# ---------------------------------------------------------------------------
# The C host over peer memory (include/b200ep.h).  G ranks live in this process on one GPU,
# connected by plain pointers; the phases run in lockstep (phase p of every rank before
# phase p + 1 of any), so every flag is already raised when its wait starts.
# ---------------------------------------------------------------------------
import ctypes as C


class _EpRanks:
    def __init__(self, dc, G, T_max, d, E, ne, K, SH, wkind, capacity=0):
        from gpu_util import pkg
        self.lib, self.G, self.d = pkg.lib(), G, d
        self.keep = []
        self.h = []
        for r in range(G):
            h = C.c_void_p()
            self.lib.b200_ep_create(C.byref(h), r, G, d, E, ne, K, SH, wkind, T_max, capacity)
            sh = [ep.shard_experts(dc[k], ne, r, G) for k in ("gates", "ups", "downs")]
            self.keep.append(sh)
            self.lib.b200_ep_set_weights(h, dc["router_w"], dc["router_bias"], sh[0], sh[1], sh[2], dc["sh_g"], dc["sh_u"],
                                         dc["sh_d"])
            self.h.append(h)
        arr = (C.c_void_p * G)(*[h.value for h in self.h])
        for h in self.h:
            self.lib.b200_ep_connect_local(h, arr)

    def forward(self, x):
        T = x.shape[0]
        for phase in range(4):
            for h in self.h:
                self.lib.b200_ep_phase(h, phase, x, T)
        outs, idxs = [], []
        for h in self.h:
            p, n = C.c_void_p(), C.c_int()
            self.lib.b200_ep_output(h, C.byref(p))
            o = torch.empty((T, self.d), device="cuda")
            self.lib.b200_copy(o, 1, p.value, 1, T * self.d * 4)
            outs.append(o)
            pi = C.c_void_p()
            self.lib.b200_ep_routing(h, C.byref(pi), None, C.byref(n))
            K = self.K
            i = torch.empty((n.value, K), dtype=torch.int32, device="cuda")
            if n.value:
                self.lib.b200_copy(i, 1, pi.value, 1, n.value * K * 4)
            idxs.append(i)
        torch.cuda.synchronize()
        return outs, torch.cat(idxs, 0)

    def close(self):
        for h in self.h:
            self.lib.b200_ep_destroy(h)


@pytest.mark.parametrize("G", [1, 2, 8])
def test_peer_memory_host_with_ranks_in_one_process(oracle, G):
    """Config-3 shape; several passes of different sizes through the same buffers (the epoch
    flags must tell them apart), a ragged token count, fewer tokens than ranks."""
    from gpu_util import dev, fp16_close, host, pkg
    d, E, ne, K, SH, wkind = 1536, 512, 64, 6, 1024, 3
    c, dc = _dev_case(oracle, 11, 200, d, E, ne, K, SH, wkind)
    sizes = (200, 77, 3, 200) + ((4096,) if G == 8 else ())     # 4096 / 8: a slice the shared expert's GEMM could cut along K
    ranks = _EpRanks(dc, G, max(sizes), d, E, ne, K, SH, wkind)
    ranks.K = K
    r = np.random.default_rng(5)
    for T in sizes:
        x = dev(r.standard_normal((T, d)).astype(np.float32))
        outs, idx = ranks.forward(x)
        want, want_idx = _single_gpu_layer(dict(dc, x=x), T, d, E, ne, K, SH, wkind)
        assert np.array_equal(host(idx), want_idx)
        for o in outs:                                   # every rank holds the whole output
            if T * K > 12 * ne:   # the same tensor-core kernels, the same order of additions: identical bits
                assert np.array_equal(host(o).view(np.uint32), want.view(np.uint32))
            else:            # a decode-sized batch takes the single GPU's fp32 few-token kernels instead
                fp16_close(host(o), want)
                assert np.array_equal(host(o), host(outs[0]))
    assert pkg.lib().raw("b200_stream_status") == 0
    ranks.close()


def test_peer_memory_host_capacity_overflow_is_reported(oracle):
    """A per-pair capacity below what the routing sends: the pass completes (rows beyond the
    capacity are dropped) and the status word reports it."""
    from gpu_util import pkg
    d, E, ne, K, SH, wkind = 256, 256, 8, 2, 256, 3
    c, dc = _dev_case(oracle, 3, 64, d, E, ne, K, SH, wkind)
    ranks = _EpRanks(dc, 2, 64, d, E, ne, K, SH, wkind, capacity=4)
    ranks.K = K
    ranks.forward(dc["x"])
    assert pkg.lib().raw("b200_stream_status") != 0
    assert pkg.lib().raw("b200_stream_status") == 0          # cleared by the read
    ranks.close()


def test_peer_memory_host_wait_runs_out(oracle):
    """A rank whose peers never dispatch: its bounded wait gives up, the kernel returns, the
    status word says so and the library stays usable."""
    from gpu_util import B200Error, pkg
    lib = pkg.lib()
    d, E, ne, K, SH, wkind = 256, 256, 8, 2, 256, 3
    c, dc = _dev_case(oracle, 3, 64, d, E, ne, K, SH, wkind)
    ranks = _EpRanks(dc, 2, 64, d, E, ne, K, SH, wkind)
    ranks.K = K
    lib.b200_ep_set_spin_limit(ranks.h[0], 2000)
    lib.b200_ep_phase(ranks.h[0], 0, dc["x"], 64)            # rank 1 never runs phase 0
    lib.b200_ep_phase(ranks.h[0], 1, dc["x"], 64)
    assert lib.raw("b200_stream_status") != 0
    assert lib.raw("b200_stream_status") == 0
    # a complete pass afterwards is clean: rank 1 catches up with the same epoch
    lib.b200_ep_phase(ranks.h[1], 0, dc["x"], 64)
    for phase in (1, 2, 3):
        for h in ranks.h:
            lib.b200_ep_phase(h, phase, dc["x"], 64)
    torch.cuda.synchronize()
    assert lib.raw("b200_stream_status") == 0
    ranks.close()
