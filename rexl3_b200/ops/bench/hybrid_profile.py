"""Two decode steps at batch N then two at batch 1 on a one-period slice of a hybrid config (e.g. three delta-net layers + one attention
layer of gdn-hybrid-27b), eager launches, between cudaProfilerStart/Stop.

    python rexl3_b200/ops/bench/hybrid_profile.py gdn-hybrid-27b 16
"""
import dataclasses
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))))
from rexl3_b200.engine import Engine, Request  # noqa: E402
from rexl3_b200.engine.gpu_backend import HybridGpuBackend  # noqa: E402
from rexl3_b200.models import hybrid  # noqa: E402
from rexl3_b200.sampling import GREEDY  # noqa: E402

name = sys.argv[1] if len(sys.argv) > 1 else "gdn-hybrid-27b"
B = int(sys.argv[2]) if len(sys.argv) > 2 else 16
base = hybrid.CONFIGS[name]
period = next(p for p in range(1, len(base.pattern) + 1) if base.pattern == base.pattern[:p] * (len(base.pattern) // p) and len(base.pattern) % p == 0)
cfg = dataclasses.replace(base, n_layers=period, pattern=base.pattern[:period], name=f"{name}-{period}L")
P = 512
bps = (P + 64) // 64 + 2
m = hybrid.HybridGPU(cfg, num_pages=(B + 1) * bps, max_rows=256, max_seqs=B + 1, max_blocks_per_seq=bps, max_prefill_rows=P)
be = HybridGpuBackend(m, max_slots=B + 1, use_graphs=False)
eng = Engine(be, None, window_rows=B, prefill_chunk=P, spec="none", prefill_policy="serial")
rng = np.random.default_rng(0)
eng.pause_decode = True
for i in range(B):
    eng.submit(Request(f"s{i}", rng.integers(0, cfg.vocab, size=P).tolist(), 40, GREEDY))
    while eng.seqs.get(f"s{i}") is None or eng.seqs[f"s{i}"].generated == 0:
        eng.step()
eng.pause_decode = False
for _ in range(2):
    eng.step()
torch.cuda.synchronize()
torch.cuda.profiler.start()
for _ in range(2):
    eng.step()
torch.cuda.synchronize()
for i in range(1, B):
    eng.cancel(f"s{i}")
for _ in range(2):
    eng.step()
torch.cuda.synchronize()
torch.cuda.profiler.stop()
print("ok", cfg.pattern)
