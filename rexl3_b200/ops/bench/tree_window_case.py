"""A verify window of draft trees against a chain window, on a 2-layer slice of the 27B config: `--seqs` sequences of `--ctx` cached tokens; the
chain window feeds [last, d1..d4] per sequence (5 rows each), the tree window feeds the anchor and 8 nodes (first chain of 4, three second
candidates and one child under a second candidate: 9 rows each, 4 of them in private pages).  CUDA-event time per window (median of
`--iters`, graphs as the engine uses them unless `--graphs 0`), and with `--profile` the windows run once between cudaProfilerStart / Stop
for a launch list."""
import argparse, dataclasses, os, sys
import numpy as np
import torch
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))))
from rexl3_b200.engine import RowRequest, TreeRequest
from rexl3_b200.engine.gpu_backend import DenseGpuBackend
from rexl3_b200.models import dense

ap = argparse.ArgumentParser()
ap.add_argument("--seqs", type=int, default=16)
ap.add_argument("--ctx", type=int, default=4096)
ap.add_argument("--iters", type=int, default=9)
ap.add_argument("--graphs", type=int, default=1)
ap.add_argument("--profile", action="store_true")
a = ap.parse_args()
cfg = dataclasses.replace(dense.CONFIGS["dense-27b"], n_layers=2, name="dense-27b-2L")
B, P = a.seqs, a.ctx
bps = (P + 128) // 64 + 2
m = dense.DenseGPU(cfg, num_pages=(B + 1) * bps + 8 * B, max_rows=256, max_seqs=B + 1, max_blocks_per_seq=bps, max_prefill_rows=min(P, 8192))
be = DenseGpuBackend(m, max_slots=B + 1, use_graphs=bool(a.graphs) and not a.profile)
rng = np.random.default_rng(0)
for s in range(B):
    toks = rng.integers(0, cfg.vocab, size=P - 1).tolist()
    for c in range(0, P - 1, 8192):
        be.prefill_slice(s, c, toks[c:c + 8192], 1, False)
PARENTS = [-1, 0, 1, 2, 3, 0, 1, 2, 5]          # rows 1-4: the first chain; 5, 6, 7: second candidates at depths 1, 2, 3; 8: a child of 5
draws = lambda n: rng.integers(0, cfg.vocab, size=n).tolist()  # noqa: E731


def chain():
    out = be.step([RowRequest(s, draws(5), P - 1) for s in range(B)], 1)
    for s in range(B):
        be.commit(s, 0)
    return out


def tree():
    out = be.step_tree([TreeRequest(s, draws(9), PARENTS, P - 1) for s in range(B)], 1)
    for s in range(B):
        be._drop_private(s)          # nothing is kept: the slot stays at P - 1 tokens for the next window
        be.pending[s] = 0
    return out


def timed(fn):
    for _ in range(3):
        fn()
    ts = []
    for _ in range(a.iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return float(np.median(ts))


if a.profile:
    chain(), tree()
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    chain()
    tree()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print("ok")
else:
    tc, tt = timed(chain), timed(tree)
    st = be.stats()
    print(f"2 layers + head, {B} seqs x ctx {P}: chain window {5 * B} rows {tc:.3f} ms; tree window {9 * B} rows {tt:.3f} ms "
          f"({st['tree_copies'] // st['tree_windows']} row-copy runs per window); host staging included (graphs {'on' if be.use_graphs else 'off'})")
