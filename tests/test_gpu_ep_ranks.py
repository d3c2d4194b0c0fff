"""The peer-memory expert-parallel host on real ranks: one process per GPU, rows over NVLink,
every rank's output compared bit for bit with the single-GPU layer (tests/ep_rank_worker.py).
Needs at least two GPUs; on a single-GPU box the same device code is covered by the
ranks-in-one-process tests of tests/test_gpu_ep.py."""
import os
import subprocess
import sys
import tempfile

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_real_ranks_equal_the_single_gpu_layer(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs, this box has {torch.cuda.device_count()}")
    with tempfile.TemporaryDirectory(prefix="b200ep_") as rdv:
        procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "ep_rank_worker.py"), str(r), str(world), rdv],
                                  stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
        outs = []
        for p in procs:
            try:
                out, _ = p.communicate(timeout=600)
            except subprocess.TimeoutExpired:
                p.kill()
                out, _ = p.communicate()
                out += "\n[timed out]"
            outs.append(out)
        for r, (p, out) in enumerate(zip(procs, outs)):
            assert p.returncode == 0, f"rank {r} failed:\n{out[-3000:]}"
