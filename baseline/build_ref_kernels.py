"""Compile the reference's CUDA sources, UNCHANGED, for sm_100 into ``baseline/_ref/libgbkernels.so``.

The reference's engine is a Rust workspace that cannot be built offline, but its kernels are self-contained
C-ABI translation units (crates/cuda/csrc/common.cuh:1-12).  This script runs nvcc on the files in place with the
flags of the reference's own build script (crates/cuda/build.rs:19: ``-O3 --std=c++17 -Xcompiler -fPIC -lineinfo -I csrc``
plus each file's ``// gb-nvcc:`` first-line flags, build.rs:134-141) and only swaps the architecture
(``-arch=sm_100`` instead of ``sm_121``, build.rs:161,209).  Nothing of this repository is compiled into the
library; it is the same-box kernel-level comparator of ``baseline/ref_kernels_bench.py``.

    python baseline/build_ref_kernels.py [--reference DIR]   # DIR defaults to $REXL3_REFERENCE_DIR
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "libgbkernels.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
# the translation units the comparator drives (each is standalone; more can be appended)
FILES = ["exl3_linear.cu"]
BASE_FLAGS = ["-O3", "--std=c++17", "-Xcompiler", "-fPIC", "-lineinfo"]


def file_flags(path: str) -> list[str]:
    first = open(path).readline()
    return first[len("// gb-nvcc:"):].split() if first.startswith("// gb-nvcc:") else []


def build(reference: str) -> str:
    csrc = os.path.join(reference, "crates", "cuda", "csrc")
    os.makedirs(OUT_DIR, exist_ok=True)
    objs = []
    for f in FILES:
        src = os.path.join(csrc, f)
        obj = os.path.join(OUT_DIR, f[:-3] + ".o")
        cmd = [NVCC, "-c", *BASE_FLAGS, "-I", csrc, "-arch=sm_100", *file_flags(src), "-o", obj, src]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stderr}")
        objs.append(obj)
    r = subprocess.run([NVCC, "-shared", "-o", OUT, *objs, "-lcublas", "-lcublasLt", "-lcudart"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stderr}")
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("REXL3_REFERENCE_DIR", ""))
    a = ap.parse_args()
    if not a.reference or not os.path.isdir(a.reference):
        sys.exit("give the reference checkout with --reference DIR or REXL3_REFERENCE_DIR")
    print(build(a.reference))
