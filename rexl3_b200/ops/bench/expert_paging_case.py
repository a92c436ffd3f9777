"""What paging the routed experts costs a decode step: a MoE GQA decoder (8 layers, d_model 1024, 32 experts of FFN 512, top-4, EXL3 3.0 bpw,
random host weights) run resident, paged with a slab that holds every expert (all hits after the first pass), and paged with a slab of
`--slots` records (evictions and file reads every step).  `--batch` sequences of `--ctx` cached tokens, one decode row each; CUDA-event time
per step (median of `--iters`), no graphs in any mode (a paged layer reads its picks on the host), the file in `--dir` (page cache warm)."""
import argparse, dataclasses, os, sys, tempfile
import numpy as np
import torch
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))))
from rexl3_b200.engine import RowRequest
from rexl3_b200.engine.gpu_backend import DenseGpuBackend
from rexl3_b200.models import expert_paging as xp
from rexl3_b200.models import moe
from rexl3_b200.sched import expert_cache as ec

ap = argparse.ArgumentParser()
ap.add_argument("--batch", type=int, default=8)
ap.add_argument("--ctx", type=int, default=512)
ap.add_argument("--iters", type=int, default=15)
ap.add_argument("--slots", type=int, default=96)
ap.add_argument("--dir", default=None)
a = ap.parse_args()
cfg = dataclasses.replace(moe.CONFIGS["test-moe"], n_layers=8, d_model=1024, n_q=8, n_kv=2, ffn=512, vocab=4096, n_experts=32, top_k=4, expert_ffn=512,
                          name="moe-paging-case")
w = moe.random_moe_weights(cfg, seed=0)
B, P = a.batch, a.ctx
kw = dict(num_pages=(B + 1) * (P // 64 + 2), max_rows=64, max_seqs=B + 1, max_blocks_per_seq=P // 64 + 2, max_prefill_rows=P)
folder = a.dir or tempfile.mkdtemp()
lay = xp.write_records(w, os.path.join(folder, "experts.records"))
rec = (lay.expert_bytes + ec.PAGE - 1) // ec.PAGE * ec.PAGE
rng = np.random.default_rng(1)
prompts = [rng.integers(0, cfg.vocab, size=P - 1).tolist() for _ in range(B)]


def run(model):
    be = DenseGpuBackend(model, max_slots=B + 1, use_graphs=False)
    for s in range(B):
        be.prefill_slice(s, 0, prompts[s], 1, False)
    pos, ts = P - 1, []
    for it in range(3 + a.iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        out = be.step([RowRequest(s, [int(rng.integers(0, cfg.vocab))], pos) for s in range(B)], 1)
        e1.record()
        torch.cuda.synchronize()
        for s in range(B):
            be.commit(s, 1)
        pos += 1
        if it >= 3:
            ts.append(e0.elapsed_time(e1))
    return float(np.median(ts)), be.stats()


t_res, _ = run(moe.MoEGPU(w, **kw))
total = cfg.n_layers * cfg.n_experts
t_all, st_all = run(moe.MoEGPU(w, expert_paging=dict(path=lay.path, budget_bytes=(total + 1) * rec), **kw))
t_few, st_few = run(moe.MoEGPU(w, expert_paging=dict(path=lay.path, budget_bytes=a.slots * rec + 1), **kw))
print(f"decode step, batch {B} x ctx {P}, {cfg.n_layers} layers x {cfg.n_experts} experts top-{cfg.top_k} ({lay.expert_bytes} B per expert record): "
      f"resident {t_res:.3f} ms; paged, slab of {total} records (all hits) {t_all:.3f} ms; paged, slab of {a.slots} records {t_few:.3f} ms "
      f"(cold rate {st_few['expert_cold_rate']:.2f}, {st_few['expert_bytes_read'] / 1e6:.1f} MB read, {st_few['expert_evictions']} evictions)")
