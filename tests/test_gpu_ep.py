"""Expert parallelism on real GPUs: N ranks (NCCL all-to-allv, and the library's peer-memory
exchange) against the single-GPU layer.
Skipped on a box with one GPU."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("mode", ["nccl", "peer"])
@pytest.mark.parametrize("fmt,T", [(0, 16), (1, 64), (2, 1024)])
def test_ep_matches_single_gpu(fmt, T, mode):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    world = 4 if n >= 4 else 2
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "tests", "ep_gpu_worker.py"), str(fmt), str(T), mode]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
