"""One layer of the 27B-class dense model as TWO tensor-parallel shards stepped phase by phase on one GPU (loopback arenas): a 2048-row
prefill slice (GEMM epilogue reduce-scatter, finish_rs, norm_rot_push, all-gather-fed GEMM) and a 64-row decode window (one-shot
all-reduce).  A small fixed case for one profiler capture of the fused compute+collective kernels; with `--time` it prints CUDA-event
timings of the reduce-scatter GEMM against the same GEMM without the collective epilogue."""
import dataclasses
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))))
from rexl3_b200.models import dense, dense_tp  # noqa: E402
from rexl3_b200.ops import kernels as K  # noqa: E402
from rexl3_b200.parallel.symm import LoopbackGroup  # noqa: E402

R = int(os.environ.get("RX_TP_CASE_RANKS", "2"))     # shards stepped on this one GPU
ROWS = 2048
DECODE_ONLY = "--decode-profile" in sys.argv            # launch-list mode: profiler range around two 64-row windows at 8192-token contexts
cfg = dataclasses.replace(dense.CONFIGS["dense-27b"], n_layers=1, vocab=8192, name="dense-27b-1L")
g = LoopbackGroup(dense_tp.DenseTPShard.layout(cfg, R, ROWS))
shards = [dense_tp.DenseTPShard(cfg, g, r, 64, ROWS, 64 if DECODE_ONLY else 4, 130 if DECODE_ONLY else 40, None, seed=1) for r in range(R)]
i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")  # noqa: E731
bt = torch.zeros(4, 40, dtype=torch.int32, device="cuda")
bt[0, :33] = torch.arange(33, dtype=torch.int32, device="cuda")
pos = list(range(ROWS))
pf = dict(seq_ids=i32([0]), q_start=i32([0]), q_len=i32([ROWS]), pos0=i32([0]), nseq=1, max_qlen=ROWS)
args = (i32([p % cfg.vocab for p in pos]), i32(pos), i32(pos), i32([0] * ROWS), i32([p + 1 for p in pos]), bt)


def run(a, **kw):
    gens = [s.phases(*a, **kw) for s in shards]
    for fns in zip(*gens):
        for fn in fns:
            fn()
    torch.cuda.synchronize()
    for s in shards:
        K.check_status(s.status, "tp case")


for _ in range(2):
    run(args, prefill=pf, want_logits=False)
d = 64
if DECODE_ONLY:
    bt2 = torch.zeros(64, 130, dtype=torch.int32, device="cuda")
    bt2[:] = torch.arange(130, dtype=torch.int32, device="cuda") % 64     # pages are shared: only the traffic pattern matters here
    a2 = (i32(list(range(d))), i32([8191] * d), i32([63] * d), i32(list(range(d))), i32([8192] * d), bt2)
    run(a2, max_ctx=8192, want_logits=False)
    torch.cuda.profiler.start()
    for _ in range(2):
        run(a2, max_ctx=8192, want_logits=False)
    torch.cuda.profiler.stop()
    print("ok")
    sys.exit(0)
a2 = (i32(list(range(d))), i32([ROWS] * d), i32([ROWS + 0] * d), i32([0] * d), i32([ROWS + 1] * d), bt)
for _ in range(2):
    run(a2, max_ctx=4096, want_logits=False)
if "--time" in sys.argv:
    s0 = shards[0]
    L = s0.layers[0]
    xr = (torch.randn(ROWS, s0.F, device="cuda") * 0.5).to(torch.float16)
    sd = s0.splits[("prefill", "down")]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    part = torch.empty(sd * ROWS * cfg.d_model, dtype=torch.float32, device="cuda")
    for name, fn in (("plain", lambda: K.exl3_gemm(xr, L["down"], part, sd, s0.status)),
                     ("reduce-scatter epilogue", lambda: s0._gemm(xr, L["down"], g.part_ptr(0, 1), sd, g.gemm_rs(0, 1, 2, sd, ROWS)))):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(10):
            fn()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 100
        fl = 2.0 * ROWS * s0.F * cfg.d_model
        print(f"down_proj shard K={s0.F} N={cfg.d_model} rows={ROWS} {name}: {us:.1f} us = {fl / us / 1e6:.0f} TFLOP/s")
print("ok")
