"""Expert parallelism over real GPUs: the sharded layer must reproduce the single-GPU layer bit for bit.

Needs two GPUs in one box; skipped otherwise (the protocol itself is covered on CPU over gloo in
test_expert_parallel_cpu.py). The ranks are child processes launched the way the benchmark is."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _gpu_count() -> int:
    import torch

    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_layer_matches_single_gpu_layer(world):
    if _gpu_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), str(ROOT / "tests" / "ep_gpu_worker.py")]
    done = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=240)
    assert done.returncode == 0, done.stdout[-4000:] + done.stderr[-4000:]
    assert done.stdout.count("parity ok") == 10 * world  # two expert paths x five exchange forms per rank
    assert done.stdout.count("overflow noticed") == 2 * world
