"""Expert-parallel MoE layer: one process per GPU, experts sharded, tokens exchanged
with all-to-all over NCCL (NVLink / NVSwitch) through torch.distributed.

Only the MoE layer shards; everything around it runs replicated, so the layer takes
the replicated activations x [T, d] and returns the replicated output [T, d]:

  * expert e lives on rank e // (ne / G); the router and the shared expert are
    replicated;
  * rank r owns the token slice [r*T/G, (r+1)*T/G): it routes the slice, packs one
    fp16 row per (token, k) slot sorted by expert - which makes the rows bound for
    each rank contiguous - and sends them (all-to-all-v);
  * the owner runs its experts on the rows it received, one GEMM group per
    (source rank, local expert) block in arrival order (no re-sort), and sends the
    fp32 results back along the same splits;
  * the token's owner adds the shared expert and the K weighted expert outputs in k
    order, and an all-gather replicates the slices.

Routing and the permutation are the single-GPU kernels on the rank's own tokens, so
top-k indices and slot order are bit-identical to the single-GPU layer; the
combination order is fixed, so results are run-to-run bit-stable.

The compute steps come from a backend object.  `CudaBackend` binds the C ABI
(b200_moe_route / _dispatch_pack / _experts_rows / _shared_combine); the tests drive
the same exchange logic on CPU (gloo) with a checker backend.  There is no CPU
fallback in this module: without the CUDA library `CudaBackend()` raises.
"""
import torch
import torch.distributed as dist


class CudaBackend:
    """Device compute through the C ABI; torch only allocates the buffers."""

    def __init__(self):
        from . import capi
        self.lib = capi.lib()

    def route(self, x, router_w, router_bias, ne, K):
        n, d = x.shape
        idx = torch.empty((n, K), dtype=torch.int32, device=x.device)
        w = torch.empty((n, K), dtype=torch.float32, device=x.device)
        if n:
            self.lib.b200_moe_route(x, router_w, router_bias, None, idx, w, n, d, ne, K)
        return idx, w

    def dispatch_pack(self, x, idx, ne):
        n, d = x.shape
        K = idx.shape[1]
        rows = torch.empty((n * K, d), dtype=torch.float16, device=x.device)
        inv = torch.empty(n * K, dtype=torch.int32, device=x.device)
        offsets = torch.zeros(ne + 1, dtype=torch.int32, device=x.device)
        if n:
            self.lib.b200_moe_dispatch_pack(x, idx, n, d, ne, K, rows, inv, offsets)
        return rows, inv, offsets

    def experts_rows(self, rows, offsets, group_map, gates, ups, downs, n_local, d, E, qkind, y=None):
        """y (optional): a [R, d] fp32 buffer to write into; rows outside the groups are left as they are."""
        R = rows.shape[0]
        if y is None:
            y = torch.empty((R, d), dtype=torch.float32, device=rows.device)
        if R:
            self.lib.b200_moe_experts_rows(rows, offsets, group_map, group_map.numel(), R, gates, ups, downs, n_local,
                                           y, d, E, qkind)
        return y

    def shared_combine(self, x, sh, y, inv, w, K, SH, qkind):
        n, d = x.shape
        out = torch.empty((n, d), dtype=torch.float32, device=x.device)
        if n:
            g, u, dn = sh if sh is not None else (None, None, None)
            self.lib.b200_moe_shared_combine(x, g, u, dn, y, inv, w, out, n, d, K, SH if sh is not None else 0, qkind)
        return out


def token_slice(T, rank, world):
    """Tokens [lo, hi) owned by `rank`."""
    return rank * T // world, (rank + 1) * T // world


def expert_owner_blocks(ne, world):
    if ne % world:
        raise ValueError(f"{ne} experts do not divide over {world} ranks")
    return ne // world


class ExpertParallelMoE:
    """gates / ups / downs hold only this rank's experts ([n_local*E, d], [n_local*E, d],
    [n_local*d, E] in the storage form named by qkind); router_w, router_bias and the
    shared expert `sh = (sh_gate, sh_up, sh_down)` (or None) are replicated."""

    def __init__(self, d, E, ne, K, SH, qkind, router_w, router_bias, gates, ups, downs, sh, group=None, backend=None):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.d, self.E, self.ne, self.K, self.SH, self.qkind = d, E, ne, K, SH, qkind
        self.n_local = expert_owner_blocks(ne, self.world)
        self.router_w, self.router_bias = router_w, router_bias
        self.gates, self.ups, self.downs, self.sh = gates, ups, downs, sh
        self.backend = backend if backend is not None else CudaBackend()
        self.last_counts = None            # rows sent to each rank by the last forward (host list)

    # -- the two exchange helpers ---------------------------------------------------
    def _all_to_all(self, send, send_rows, recv_rows):
        recv = torch.empty((sum(recv_rows),) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
        if self.world == 1:
            recv.copy_(send)
        else:
            dist.all_to_all_single(recv, send.contiguous(), list(recv_rows), list(send_rows), group=self.group)
        return recv

    def _gather_slices(self, part, T):
        if self.world == 1:
            return part
        longest = max(token_slice(T, r, self.world)[1] - token_slice(T, r, self.world)[0] for r in range(self.world))
        pad = torch.zeros((longest, self.d), dtype=part.dtype, device=part.device)
        pad[:part.shape[0]] = part
        full = torch.empty((self.world * longest, self.d), dtype=part.dtype, device=part.device)
        dist.all_gather_into_tensor(full, pad, group=self.group)
        pieces = []
        for r in range(self.world):
            lo, hi = token_slice(T, r, self.world)
            pieces.append(full[r * longest:r * longest + (hi - lo)])
        return torch.cat(pieces, 0)

    # -- the layer --------------------------------------------------------------------
    def forward(self, x):
        T = x.shape[0]
        G, nl, be = self.world, self.n_local, self.backend
        lo, hi = token_slice(T, self.rank, G)
        xs = x[lo:hi].contiguous()
        idx, w = be.route(xs, self.router_w, self.router_bias, self.ne, self.K)
        rows, inv, offsets = be.dispatch_pack(xs, idx, self.ne)
        counts = (offsets[1:] - offsets[:-1]).to(torch.int32)              # rows per expert, [ne] = [G, nl]
        recv_counts = torch.empty_like(counts)                             # [G sources, nl]
        if G == 1:
            recv_counts.copy_(counts)
        else:
            dist.all_to_all_single(recv_counts, counts, group=self.group)
        both = torch.stack([counts.view(G, nl).sum(1), recv_counts.view(G, nl).sum(1)]).cpu()   # the one host sync
        send_rows, recv_rows = both[0].tolist(), both[1].tolist()
        self.last_counts = send_rows
        got = self._all_to_all(rows, send_rows, recv_rows)
        # one group per (source rank, local expert) block, in arrival order
        goff = torch.zeros(G * nl + 1, dtype=torch.int32, device=x.device)
        goff[1:] = torch.cumsum(recv_counts, 0)
        gmap = torch.arange(nl, dtype=torch.int32, device=x.device).repeat(G)
        y_remote = be.experts_rows(got, goff, gmap, self.gates, self.ups, self.downs, nl, self.d, self.E, self.qkind)
        y = self._all_to_all(y_remote, recv_rows, send_rows)
        part = be.shared_combine(xs, self.sh, y, inv, w, self.K, self.SH, self.qkind)
        return self._gather_slices(part, T), idx

    def forward_reduce(self, x):
        """The same layer without any dispatch.  The activations are replicated, so every rank
        routes all T tokens (identical indices everywhere), runs only ITS experts on the slots
        that hit them, and forms a partial output: the weighted sum of its experts' results
        for every token, plus the shared expert for the tokens of its own slice.  One
        all-reduce adds the partials.  No split sizes travel and the host reads nothing, at
        the price of routing every token on every rank and of an output-sized reduction
        ([T, d] fp32) instead of two row exchanges.  The K expert outputs of a token are added
        per rank first, so the result equals forward()'s up to the order of those additions."""
        T = x.shape[0]
        G, nl, be, K = self.world, self.n_local, self.backend, self.K
        if G > 1 and dist.is_initialized() and T % G == 0 and T > 0:
            # routing is per token: each rank routes its slice and the (small) results are gathered
            lo, hi = token_slice(T, self.rank, G)
            idx_s, w_s = be.route(x[lo:hi], self.router_w, self.router_bias, self.ne, K)
            idx = torch.empty((T, K), dtype=idx_s.dtype, device=x.device)
            w = torch.empty((T, K), dtype=w_s.dtype, device=x.device)
            dist.all_gather_into_tensor(idx, idx_s.contiguous(), group=self.group)
            dist.all_gather_into_tensor(w, w_s.contiguous(), group=self.group)
        else:
            idx, w = be.route(x, self.router_w, self.router_bias, self.ne, K)
        rows, inv, offsets = be.dispatch_pack(x, idx, self.ne)
        e0 = self.rank * nl
        key = (rows.shape[0], x.device)
        if getattr(self, "_y_key", None) != key:
            # persistent and zero-initialised: rows no local expert writes in a call keep finite
            # values (zeros, or results of earlier calls), so a weight of 0 masks them exactly
            self._y_buf = torch.zeros((rows.shape[0], self.d), dtype=torch.float32, device=x.device)
            self._y_key = key
        gmap = torch.arange(nl, dtype=torch.int32, device=x.device)
        y = be.experts_rows(rows, offsets[e0:e0 + nl + 1].contiguous(), gmap, self.gates, self.ups, self.downs, nl, self.d,
                            self.E, self.qkind, y=self._y_buf)
        w_local = torch.where((idx >= e0) & (idx < e0 + nl), w, torch.zeros_like(w))
        lo, hi = token_slice(T, self.rank, G)
        parts = []
        for a, b, sh in ((0, lo, None), (lo, hi, self.sh), (hi, T, None)):
            if b > a:
                parts.append(be.shared_combine(x[a:b], sh, y, inv[a * K:b * K], w_local[a:b], K, self.SH, self.qkind))
        out = parts[0] if len(parts) == 1 else torch.cat(parts, 0)
        return self._reduce(out), idx

    def graphed_reduce(self, x):
        """forward_reduce() for inputs of x's shape, captured once into a CUDA graph (the
        dispatch-free form reads nothing on the host and has static shapes, so the whole layer -
        kernels, the small torch ops between them and the NCCL all-reduce - replays as one
        launch).  Returns replay(x_new) -> (out, idx); the tensors it returns are reused by the
        next replay.  CUDA backend only."""
        lib = self.backend.lib
        side = torch.cuda.Stream(device=x.device)
        static_x = x.clone()
        side.wait_stream(torch.cuda.current_stream(x.device))
        lib.b200_set_stream(side.cuda_stream)
        try:
            with torch.cuda.stream(side):
                for _ in range(2):                       # grows workspaces, builds tensor maps, warms NCCL
                    self.forward_reduce(static_x)
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                out, idx = self.forward_reduce(static_x)
        finally:
            lib.b200_set_stream(None)
        torch.cuda.current_stream(x.device).wait_stream(side)

        def replay(x_new):
            static_x.copy_(x_new)
            graph.replay()
            return out, idx

        return replay

    def _reduce(self, partial):
        """Sum of the ranks' partial outputs (in place)."""
        if self.world > 1:
            dist.all_reduce(partial, group=self.group)
        return partial


def shard_experts(t, ne, rank, world):
    """Rows of a stacked expert tensor ([ne*rows_per_expert, ...] or packed bytes of
    that matrix) that belong to `rank`."""
    nl = expert_owner_blocks(ne, world)
    per = t.shape[0] // ne
    return t[rank * nl * per:(rank + 1) * nl * per].contiguous()
