"""Multi-GPU paths (need at least two GPUs; skipped otherwise): head-sharded decode with
the peer-memory all-gather of per-head results, checked against the library all-gather
and against the unsharded result."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_head_sharded_decode_with_peer_memory_gather():
    world = 4 if torch.cuda.device_count() >= 4 else 2
    child = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_head_gather_child.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                          f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                          "--master-port", "29541", child],
                         env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and res.stdout.count("OK") == world, res.stdout[-2000:] + res.stderr[-4000:]
