"""Builds goinfer_b200/libgoinfer_b200.so from csrc/*.cu with nvcc for sm_100a, in-tree.

nvcc cross-compiles without a GPU. Objects are cached in csrc/build/ by source modification time.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_DIR, "csrc")
OUT = os.path.join(_DIR, "libgoinfer_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "-ccbin", "/usr/bin/g++"]


def _newer(src: str, dst: str, deps) -> bool:
    if not os.path.exists(dst):
        return True
    t = os.path.getmtime(dst)
    return any(os.path.getmtime(d) > t for d in [src] + list(deps))


def build(verbose: bool = False, force: bool = False) -> str:
    os.makedirs(os.path.join(CSRC, "build"), exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    deps = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(_DIR, "..", "include", "*.h"))
    objs, jobs = [], []
    for s in srcs:
        o = os.path.join(CSRC, "build", os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or _newer(s, o, deps):
            cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))

    with ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(run, jobs))
    if jobs or not os.path.exists(OUT):
        run([NVCC, "-shared", "-o", OUT] + objs + ["-ccbin", "/usr/bin/g++", "-lcudart"])
    return OUT


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
