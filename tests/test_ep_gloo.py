"""Expert-parallel MoE: the exchange logic of jdm-ghassan_v1_flach_b200/ep.py on CPU,
world_size 2 and 4 over gloo, with the CPU oracle standing in for the device compute
(test infrastructure only).  Every rank must reproduce the single-process layer."""
import importlib
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cases import moe_case
from oracle_lib import OracleOnly

ep = importlib.import_module("jdm-ghassan_v1_flach_b200.ep")

D, E, NE, K, SH = 64, 32, 8, 2, 64


class CheckerBackend:
    """The four compute steps on CPU tensors through the oracle (fp32 everywhere)."""

    def __init__(self, oracle):
        self.o = oracle

    def route(self, x, router_w, router_bias, ne, K):
        if x.shape[0] == 0:
            return torch.empty((0, K), dtype=torch.int32), torch.empty((0, K))
        _, idx, w = self.o.moe_route(x.numpy(), router_w.numpy(), None if router_bias is None else router_bias.numpy(),
                                     ne, K)
        return torch.from_numpy(idx), torch.from_numpy(w)

    def dispatch_pack(self, x, idx, ne):
        n, K = idx.shape
        if n == 0:
            return torch.empty((0, x.shape[1])), torch.empty(0, dtype=torch.int32), torch.zeros(ne + 1, dtype=torch.int32)
        grouped, offsets = self.o.moe_permutation(idx.numpy(), ne)
        inv = np.empty(n * K, np.int32)
        inv[grouped] = np.arange(n * K, dtype=np.int32)
        rows = x.numpy()[grouped // K]
        return torch.from_numpy(rows.copy()), torch.from_numpy(inv), torch.from_numpy(offsets)

    def experts_rows(self, rows, offsets, group_map, gates, ups, downs, n_local, d, E, qkind, y=None):
        keep = y
        y = np.zeros((rows.shape[0], d), np.float32) if keep is None else keep.numpy()
        off, gm = offsets.numpy(), group_map.numpy()
        g3, u3, d3 = gates.numpy().reshape(n_local, E, d), ups.numpy().reshape(n_local, E, d), downs.numpy().reshape(n_local, d, E)
        for g in range(len(gm)):
            lo, hi = int(off[g]), int(off[g + 1])
            if hi > lo:
                e = int(gm[g])
                xr = rows.numpy()[lo:hi]
                act = self.o.swiglu(self.o.linear(xr, g3[e], -2, hi - lo, d, E), self.o.linear(xr, u3[e], -2, hi - lo, d, E))
                y[lo:hi] = self.o.linear(act, d3[e], -2, hi - lo, E, d)
        return torch.from_numpy(y) if keep is None else keep

    def shared_combine(self, x, sh, y, inv, w, K, SH, qkind):
        n, d = x.shape
        out = np.zeros((n, d), np.float32)
        if n and sh is not None:
            g, u, dn = (t.numpy() for t in sh)
            act = self.o.swiglu(self.o.linear(x.numpy(), g, -2, n, d, SH), self.o.linear(x.numpy(), u, -2, n, d, SH))
            out = self.o.linear(act, dn, -2, n, SH, d)
        yv, iv, wv = y.numpy(), inv.numpy(), w.numpy()
        for t in range(n):
            for k in range(K):
                out[t] = out[t] + wv[t, k] * yv[iv[t * K + k]]
        return torch.from_numpy(out.astype(np.float32))


def _case(T, seed=5):
    o = OracleOnly()
    return o, moe_case(o, seed=seed, N=T, d=D, E=E, ne=NE, K=K, SH=SH, wkind=-2, bias_sigma=0.3)


def _layer(o, c, rank, world, group=None):
    t = torch.from_numpy
    sh = (t(c["sh_g"]), t(c["sh_u"]), t(c["sh_d"]))
    return ep.ExpertParallelMoE(D, E, NE, K, SH, -2, t(c["router_w"]), t(c["router_bias"]),
                                ep.shard_experts(t(c["gates"]), NE, rank, world),
                                ep.shard_experts(t(c["ups"]), NE, rank, world),
                                ep.shard_experts(t(c["downs"]), NE, rank, world), sh, group=group,
                                backend=CheckerBackend(o))


def _want(o, c):
    out, _, idx, _ = o.moe_forward(c["x"], c["router_w"], c["router_bias"], c["gates"], c["ups"], c["downs"],
                                   c["sh_g"], c["sh_u"], c["sh_d"], D, E, NE, K, SH, -2)
    return out, idx


def _worker(rank, world, port, T, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        o, c = _case(T)
        layer = _layer(o, c, rank, world)
        out, idx = layer.forward(torch.from_numpy(c["x"]))
        want, want_idx = _want(o, c)
        lo, hi = ep.token_slice(T, rank, world)
        ok = bool(np.allclose(out.numpy(), want, rtol=1e-5, atol=1e-6)) and np.array_equal(idx.numpy(), want_idx[lo:hi])
        again, _ = layer.forward(torch.from_numpy(c["x"]))
        ok = ok and np.array_equal(out.numpy().view(np.uint32), again.numpy().view(np.uint32))
        # the dispatch-free form: every rank holds the whole output and all indices
        red, ridx = layer.forward_reduce(torch.from_numpy(c["x"]))
        ok = ok and bool(np.allclose(red.numpy(), want, rtol=1e-5, atol=1e-6)) and np.array_equal(ridx.numpy(), want_idx)
        red2, _ = layer.forward_reduce(torch.from_numpy(c["x"]))      # second call reuses the row buffer
        ok = ok and bool(np.allclose(red2.numpy(), want, rtol=1e-5, atol=1e-6))
        q.put((rank, ok, sum(layer.last_counts)))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_single_process_equals_layer():
    o, c = _case(13)
    out, idx = _layer(o, c, 0, 1).forward(torch.from_numpy(c["x"]))
    want, want_idx = _want(o, c)
    np.testing.assert_allclose(out.numpy(), want, rtol=1e-5, atol=1e-6)
    assert np.array_equal(idx.numpy(), want_idx)
    red, ridx = _layer(o, c, 0, 1).forward_reduce(torch.from_numpy(c["x"]))
    np.testing.assert_allclose(red.numpy(), want, rtol=1e-5, atol=1e-6)
    assert np.array_equal(ridx.numpy(), want_idx)


@pytest.mark.parametrize("world,T", [(2, 13), (2, 1), (4, 30), (2, 8), (4, 16)])
def test_expert_parallel_over_gloo(world, T):
    """T = 1 leaves ranks without tokens; 13 and 30 give ragged slices and ragged expert loads;
    8 and 16 divide evenly (the dispatch-free form then routes per slice and gathers the indices)."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, T, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    got = sorted(q.get(timeout=5) for _ in range(world))
    assert [g[0] for g in got] == list(range(world))
    assert all(g[1] for g in got), got
    assert sum(g[2] for g in got) == T * K          # every slot was sent exactly once


def test_token_slices_and_expert_blocks():
    for T in (0, 1, 7, 64):
        for G in (1, 2, 4, 8):
            cuts = [ep.token_slice(T, r, G) for r in range(G)]
            assert cuts[0][0] == 0 and cuts[-1][1] == T
            assert all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
    assert ep.expert_owner_blocks(64, 8) == 8
    with pytest.raises(ValueError):
        ep.expert_owner_blocks(72, 7)
