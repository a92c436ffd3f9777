"""Prefill of ONE prompt on a one-period slice of a hybrid config (e.g. three delta-net layers + one attention layer of gdn-hybrid-27b):
CUDA-event time of the slice per chunk, and the same forward once more between cudaProfilerStart/Stop for a launch list.

    python rexl3_b200/ops/bench/hybrid_prefill_case.py gdn-hybrid-27b 4096
"""
import dataclasses
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))))
from rexl3_b200.models import hybrid  # noqa: E402

name = sys.argv[1] if len(sys.argv) > 1 else "gdn-hybrid-27b"
P = int(sys.argv[2]) if len(sys.argv) > 2 else 4096
base = hybrid.CONFIGS[name]
period = next(p for p in range(1, len(base.pattern) + 1) if base.pattern == base.pattern[:p] * (len(base.pattern) // p) and len(base.pattern) % p == 0)
cfg = dataclasses.replace(base, n_layers=period, pattern=base.pattern[:period], name=f"{name}-{period}L")
blocks = P // 64 + 2
m = hybrid.HybridGPU(cfg, num_pages=blocks + 1, max_rows=64, max_seqs=2, max_blocks_per_seq=blocks, max_prefill_rows=P)
i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")  # noqa: E731
rng = np.random.default_rng(0)
ids = i32(rng.integers(0, cfg.vocab, size=P).tolist())
pos = torch.arange(P, dtype=torch.int32, device="cuda")
bt = torch.zeros(2, blocks, dtype=torch.int32, device="cuda")
bt[0] = torch.arange(blocks, dtype=torch.int32, device="cuda")
slots = (bt[0][(pos // 64).long()] * 64 + pos % 64).to(torch.int32)
seqs = torch.zeros(P, dtype=torch.int32, device="cuda")
pf = dict(seq_ids=i32([0]), q_start=i32([0]), q_len=i32([P]), pos0=i32([0]), nseq=1, max_qlen=P)


def run():
    m.forward_rows(ids, pos, slots, seqs, pos + 1, bt, prefill=pf, logit_rows=torch.tensor([P - 1], device="cuda"))


for _ in range(2):
    run()
torch.cuda.synchronize()
m.check()
e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
e0.record()
for _ in range(3):
    run()
e1.record()
torch.cuda.synchronize()
ms = e0.elapsed_time(e1) / 3
rec = sum(1 for k in cfg.pattern if k != "A")
print(f"{cfg.name}: {P}-token prefill of {period} layers ({rec} recurrent) {ms:.2f} ms = {P / ms * 1e3 / (len(base.pattern) / period):.0f} tokens/s scaled to the "
      f"{len(base.pattern)}-layer model")
torch.cuda.profiler.start()
run()
torch.cuda.synchronize()
torch.cuda.profiler.stop()
