"""ZeRO-1 on real GPUs: NCCL all-gather path and fused update+push path against
the oracle, on as many GPUs as the box has (2, 4 or 8); skipped on one GPU."""
import os
import socket
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _world():
    import torch
    n = torch.cuda.device_count()
    return 8 if n >= 8 else 4 if n >= 4 else 2 if n >= 2 else 0


@pytest.mark.parametrize("variant", [0, 1], ids=["peers_in_order", "evict_first_stores"])
def test_push_path_under_its_other_store_orders(variant):
    """The fused update+push kernel has three ways of ordering its remote stores
    (GOMETAL_PUSH_VARIANT; 2, the rotating one, is the default and runs in the test below)."""
    world = _world()
    if world == 0:
        pytest.skip("needs at least 2 GPUs")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "zero1_worker.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", OMP_NUM_THREADS="1", GM_TEST_EXCHANGES="push",
               GOMETAL_PUSH_VARIANT=str(variant))
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    for r in range(world):
        assert f"rank {r} ok" in out.stdout


def test_zero1_paths_match_oracle_on_all_ranks():
    import torch
    n = torch.cuda.device_count()
    world = 8 if n >= 8 else 4 if n >= 4 else 2 if n >= 2 else 0
    if world == 0:
        pytest.skip("needs at least 2 GPUs")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "zero1_worker.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", OMP_NUM_THREADS="1")
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    for r in range(world):
        assert f"rank {r} ok" in out.stdout
