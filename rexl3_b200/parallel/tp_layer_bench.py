"""Fused compute + collective kernels over REAL NVLink, timed on the device: two layers of the 27B-class dense model as one tensor-parallel
shard per GPU (one process per GPU), a prefill slice of `--rows` rows stepped phase by phase on every rank, CUDA events around every GEMM
launch.  For the two row-parallel projections (o_proj, down_proj: GEMM whose epilogue pushes each 128-column tile to its owner rank =
reduce-scatter) and the two column-parallel ones (qkv, gate_up: the activation producer waits for the all-gathered input rank by rank) it
prints, max over ranks: time, FLOP/s, the bytes that cross NVLink per rank and the achieved fraction of the roofline
max(FLOPs / GEMM peak, NVLink bytes / link bandwidth); and the same GEMMs run alone (no collective hooks) for comparison.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29531 -m rexl3_b200.parallel.tp_layer_bench
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import sys

import torch
import torch.distributed as dist


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=6)
    ap.add_argument("--gemm-peak-tflops", type=float, default=1654.7, help="measured cuBLAS bf16 burst of this pool")
    ap.add_argument("--link-gbs", type=float, default=770.0, help="measured peer copy bandwidth per direction")
    a = ap.parse_args()
    from ..models import dense
    from ..ops import kernels as K
    from . import runtime
    ctx = runtime.init(timeout_s=300)
    R, rank, M = ctx.world, ctx.rank, a.rows
    cfg = dataclasses.replace(dense.CONFIGS["dense-27b"], n_layers=2, vocab=8192, name="dense-27b-2L")
    blocks = M // 64 + 2
    shard, group = runtime.build_dense_tp(ctx, cfg, num_pages=blocks + 1, max_rows=M, max_slots=2, max_blocks_per_seq=blocks, seed=1)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=ctx.device)  # noqa: E731
    pos = torch.arange(M, dtype=torch.int32, device=ctx.device)
    bt = torch.zeros(2, blocks, dtype=torch.int32, device=ctx.device)
    bt[0] = torch.arange(blocks, dtype=torch.int32, device=ctx.device)
    slots = (bt[0][(pos // 64).long()] * 64 + pos % 64).to(torch.int32)
    pf = dict(seq_ids=i32([0]), q_start=i32([0]), q_len=i32([M]), pos0=i32([0]), nseq=1, max_qlen=M)
    ids = (pos % cfg.vocab).to(torch.int32)
    args = (ids, pos, slots, torch.zeros(M, dtype=torch.int32, device=ctx.device), pos + 1, bt)
    names = {}
    for L in shard.layers:
        for k in ("qkv", "o", "gate_up", "down"):
            names[id(L[k])] = k
    records = []
    inner = shard._gemm

    def timed(x, w, part_ptr, splits, desc=None):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = inner(x, w, part_ptr, splits, desc)
        e1.record()
        records.append((names.get(id(w), "other"), e0, e1, w.K, w.N, splits))
        return out
    shard._gemm = timed

    def step():
        for p in shard.phases(*args, prefill=pf, want_logits=False):
            p()
    for _ in range(2):
        step()
    torch.cuda.synchronize()
    dist.barrier(group=ctx.ctrl)
    K.check_status(shard.status, "tp layer bench")
    records.clear()
    for _ in range(a.iters):
        step()
    torch.cuda.synchronize()
    K.check_status(shard.status, "tp layer bench")
    fused = {}
    for name, e0, e1, kk, nn, s in records:
        fused.setdefault(name, []).append((e0.elapsed_time(e1), kk, nn, s))
    # the same GEMMs alone: local input, local fp32 partials, no flags
    shard._gemm = inner
    alone = {}
    L = shard.layers[1]
    for name in ("qkv", "o", "gate_up", "down"):
        w = L[name]
        s = shard.splits[("prefill", name)]
        x = (torch.randn(M, w.K, device=ctx.device) * 0.5).to(torch.float16)
        part = torch.empty(s * M * w.N, dtype=torch.float32, device=ctx.device)
        for _ in range(2):
            K.exl3_gemm(x, w, part, s, shard.status)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            K.exl3_gemm(x, w, part, s, shard.status)
        e1.record()
        torch.cuda.synchronize()
        alone[name] = e0.elapsed_time(e1) / a.iters
        del x, part
    rows = []
    for name in ("qkv", "o", "gate_up", "down"):
        ts = sorted(t for t, *_ in fused[name])
        _, kk, nn, s = fused[name][0]
        t = torch.tensor([ts[len(ts) // 2], alone[name]], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=ctx.ctrl)
        ms, ms_alone = float(t[0]), float(t[1])
        flops = 2.0 * M * kk * nn
        rs = name in ("o", "down")
        # reduce-scatter: this rank's partial of every column it does not own leaves the GPU (f32, per K split);
        # all-gather-fed: the other ranks' fp16 slices of the rotated input arrive
        link_bytes = M * nn * (R - 1) / R * 4 * s if rs else M * kk * (R - 1) / R * 2
        roof_ms = max(flops / (a.gemm_peak_tflops * 1e12), link_bytes / (a.link_gbs * 1e9)) * 1e3
        rows.append(dict(gemm=name, K=kk, N=nn, splits=s, collective="reduce-scatter epilogue" if rs else "all-gather-fed input", ms=round(ms, 4),
                         tflops=round(flops / ms / 1e9, 1), nvlink_mb_per_rank=round(link_bytes / 1e6, 1), roofline_ms=round(roof_ms, 4),
                         roofline_fraction=round(roof_ms / ms, 3), ms_without_collective=round(ms_alone, 4)))
    if rank == 0:
        print(json.dumps(dict(bench="tp_layer", ranks=R, rows=M, model=cfg.name, nvls=bool(group.mm_mc_base), gemm_peak_tflops=a.gemm_peak_tflops,
                              link_gbs=a.link_gbs, results=rows)))
    runtime.shutdown(ctx, group)
    return 0


if __name__ == "__main__":
    sys.exit(main())
