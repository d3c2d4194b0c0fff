"""One rank of the real multi-GPU check of the peer-memory expert-parallel host
(tests/test_gpu_ep_ranks.py starts one of these per GPU).  No collective library and no
torch.distributed: the ranks meet through files (b200_ep_rendezvous_dir), exchange rows over
NVLink, and each compares what it received with the single-GPU layer computed locally.

usage: python tests/ep_rank_worker.py <rank> <world> <rendezvous dir>
"""
import ctypes as C
import importlib
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path[:0] = [os.path.dirname(HERE), HERE]


def file_barrier(rdv, name, rank, world, timeout=120.0):
    open(os.path.join(rdv, f"{name}.{rank}"), "w").close()
    t0 = time.time()
    while not all(os.path.exists(os.path.join(rdv, f"{name}.{r}")) for r in range(world)):
        if time.time() - t0 > timeout:
            raise TimeoutError(f"barrier {name}: a rank is missing")
        time.sleep(0.01)


def main():
    rank, world, rdv = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    import torch
    torch.cuda.set_device(rank)
    from cases import moe_case
    from gpu_util import dev, fp16_close, host, pkg
    from oracle_lib import OracleOnly
    ep = importlib.import_module("jdm-ghassan_v1_flach_b200.ep")
    lib = pkg.lib()
    d, E, ne, K, SH, q = 1536, 512, 64, 6, 1024, 3
    T_max = 600
    c = moe_case(OracleOnly(), 11, 8, d, E, ne, K, SH, q)          # the same seeded weights on every rank
    dc = {k: dev(v) for k, v in c.items()}
    shard = [ep.shard_experts(dc[k], ne, rank, world) for k in ("gates", "ups", "downs")]
    h = C.c_void_p()
    lib.b200_ep_create(C.byref(h), rank, world, d, E, ne, K, SH, q, T_max, 0)
    lib.b200_ep_set_weights(h, dc["router_w"], dc["router_bias"], shard[0], shard[1], shard[2], dc["sh_g"], dc["sh_u"], dc["sh_d"])
    lib.b200_ep_rendezvous_dir(h, rdv.encode(), 120000)
    r = np.random.default_rng(5)
    for T in (600, 77, 3, 512, 600):
        x = dev(r.standard_normal((T, d)).astype(np.float32))       # the same tokens on every rank (same seed)
        lib.b200_ep_forward(h, x, T)
        p = C.c_void_p()
        lib.b200_ep_output(h, C.byref(p))
        got = torch.empty((T, d), device="cuda")
        lib.b200_copy(got, 1, p.value, 1, T * d * 4)
        want = torch.empty((T, d), device="cuda")
        want_idx = torch.empty((T, K), dtype=torch.int32, device="cuda")
        lib.b200_moe_forward_bias_half(x, dc["router_w"], dc["router_bias"], dc["gates"], dc["ups"], dc["downs"], dc["sh_g"],
                                       dc["sh_u"], dc["sh_d"], want, None, want_idx, None, None, None, None, T, d, E, ne, K,
                                       SH, q)
        pi, n = C.c_void_p(), C.c_int()
        lib.b200_ep_routing(h, C.byref(pi), None, C.byref(n))
        lo = rank * T // world
        if n.value:
            idx = torch.empty((n.value, K), dtype=torch.int32, device="cuda")
            lib.b200_copy(idx, 1, pi.value, 1, n.value * K * 4)
            assert torch.equal(idx, want_idx[lo:lo + n.value]), f"rank {rank} T {T}: routing differs"
        torch.cuda.synchronize()
        assert lib.raw("b200_stream_status") == 0, f"rank {rank} T {T}: a bounded wait ran out"
        if T * K > 12 * ne:          # below that the single GPU runs its fp32 decode-batch kernels
            assert torch.equal(got, want), f"rank {rank} T {T}: max diff {(got - want).abs().max().item():.3e}"
        else:
            fp16_close(host(got), host(want))
        file_barrier(rdv, f"pass{T}_{r.integers(1 << 30)}", rank, world)
    file_barrier(rdv, "done", rank, world)        # nobody unmaps while a peer may still store
    lib.b200_ep_destroy(h)
    print(f"rank {rank}: ok")


if __name__ == "__main__":
    main()
