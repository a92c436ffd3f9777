"""Build the host-side native library (``librexl3_host.so``): trellis encoder, tokenizer core, weight loader."""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "librexl3_host.so")


def build(force: bool = False) -> str:
    srcs = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cpp"))
    newest = max(os.path.getmtime(s) for s in srcs)
    if force or not os.path.exists(OUT) or os.path.getmtime(OUT) < newest:
        cmd = ["g++", "-O3", "-march=x86-64-v3", "-std=c++17", "-shared", "-fPIC", "-pthread", "-o", OUT, *srcs]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"g++ failed:\n{r.stdout}\n{r.stderr}")
    return OUT


if __name__ == "__main__":
    print(build(force=True))
