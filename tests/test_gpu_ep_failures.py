"""Failure paths of the expert-parallel layer, driven from the host over a stand-in NCCL: no GPU faults, traps or
hangs; an error code from a fake of the failing call, and bounded waits that are made to run out. The worker runs
in a child process so that the stand-in, not a framework's NCCL, is what the library binds."""
import os
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_failures_inside_the_exchange_are_reported_not_hung(tmp_path):
    gcc = shutil.which("gcc")
    cuda = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    if not gcc or not (cuda / "include" / "cuda_runtime.h").exists():
        pytest.skip("needs gcc and the CUDA runtime headers to build the stand-in")
    stub = tmp_path / "libnccl_stub.so"
    subprocess.run([gcc, "-shared", "-fPIC", "-O1", f"-I{cuda / 'include'}", str(ROOT / "tests" / "stub_nccl.c"), "-o", str(stub),
                    f"-L{cuda / 'lib64'}", "-lcudart", f"-Wl,-rpath,{cuda / 'lib64'}"], check=True)
    env = dict(os.environ, NVMOE_NCCL_LIBRARY=str(stub))
    done = subprocess.run([sys.executable, str(ROOT / "tests" / "ep_stub_worker.py"), str(stub)], cwd=ROOT, env=env,
                          capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-3000:]
    assert "all checks held" in done.stdout
