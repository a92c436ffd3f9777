"""Two decode steps of one rank's share of the MLA + MoE decoder (16 of 128 heads, 32 of 256 experts; 1 dense + 3 routed layers at the
full layer shapes) at batch N with 8192-token contexts, between cudaProfilerStart/Stop.  The latent cache holds whatever the
allocator left there: only timing is of interest."""
import dataclasses
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))))
from rexl3_b200.engine.backend import RowRequest  # noqa: E402
from rexl3_b200.engine.gpu_backend import DenseGpuBackend  # noqa: E402
from rexl3_b200.models import mla  # noqa: E402

B = int(sys.argv[1]) if len(sys.argv) > 1 else 64
P = 8192
cfg = dataclasses.replace(mla.CONFIGS["mla-moe-671b"], n_layers=4, n_dense=1, name="mla-4L")
bps = (P + 64) // 64 + 2
m = mla.MlaMoEGPU(cfg, num_pages=(B + 1) * bps, max_rows=256, max_seqs=B + 1, max_blocks_per_seq=bps, max_prefill_rows=256, heads=(0, 16), experts=(0, 32))
be = DenseGpuBackend(m, max_slots=B + 1, use_graphs=False)
for s in range(B):
    be._ensure(s, P + 8)
    be.len[s] = P
reqs = [RowRequest(s, [17 + s], P) for s in range(B)]
be.step(reqs, 8)
for s in range(B):
    be.commit(s, 0)
torch.cuda.synchronize()
torch.cuda.profiler.start()
for _ in range(2):
    be.step(reqs, 8)
    for s in range(B):
        be.commit(s, 0)
torch.cuda.synchronize()
torch.cuda.profiler.stop()
print("ok")
