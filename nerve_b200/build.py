"""Builds libnerve_cuda_moe.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m nerve_b200.build [--force] [--verbose]

The library is the product: the package refuses to run without it and has no CPU fallback.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
INCLUDE = PACKAGE_DIR.parent / "include"
LIB_PATH = PACKAGE_DIR / "libnerve_cuda_moe.so"

SOURCES = ["capi.cu", "router.cu", "schedule.cu", "quantize.cu", "experts_simt.cu", "experts_tc.cu", "reduce.cu", "probe.cu", "ffn_tail.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "--extended-lambda",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-O3",
    "-Xptxas", "-v",
]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: the CUDA MoE backend cannot be built")


def _stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h")) + [Path(__file__)]
    return any(d.stat().st_mtime > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not _stale():
        return LIB_PATH
    nvcc = nvcc_path()
    objdir = PACKAGE_DIR / "build"
    objdir.mkdir(exist_ok=True)
    env = dict(os.environ)
    # nvcc needs a host compiler it knows; the image's default CC may point elsewhere
    host = "/usr/bin/g++" if Path("/usr/bin/g++").exists() else shutil.which("g++")
    procs = []
    for src in SOURCES:
        obj = objdir / (src + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-ccbin", host, "-I", str(INCLUDE), "-c", str(CSRC / src), "-o", str(obj)]
        procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)))
    logs, objs, failed = [], [], []
    for src, obj, proc in procs:
        out, _ = proc.communicate()
        logs.append(f"==== {src}\n{out}")
        objs.append(str(obj))
        if proc.returncode != 0:
            failed.append(src)
    (objdir / "ptxas.log").write_text("\n".join(logs))
    if failed or verbose:
        sys.stderr.write("\n".join(logs) + "\n")
    if failed:
        raise RuntimeError(f"nvcc failed on {failed}")
    link = [nvcc, "-shared", "-ccbin", host, "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB_PATH), *objs, "-ldl"]
    res = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    if res.returncode != 0:
        sys.stderr.write(res.stdout)
        raise RuntimeError("link failed")
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
