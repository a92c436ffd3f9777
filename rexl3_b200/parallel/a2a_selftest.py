"""Token all-to-all expert parallelism over REAL NVLink, one process per GPU: every rank feeds its OWN sequences (data-parallel attention), a
(row, slot) pair travels to the rank that owns its expert and the result travels home (parallel/ep.py A2aComm, ops/csrc/moe.cu).

Two parts.  (1) Correctness: a small MoE whose host weights every rank draws from one seed; each rank prefills its own prompt and decodes a
few tokens through its shard, and the logits must equal, bit for bit, those of a one-GPU executor holding all the experts that the same
process runs on the same prompt.  (2) Timing: two layers of the 30B-class MoE (128 experts, top-8, d 2048), a prefill slice of `--rows` rows
per rank, CUDA events around whole forwards, max over ranks; printed beside the bytes a rank puts on NVLink per layer (dispatch bf16 rows out,
f32 results back) and the time the same slice takes on one GPU with every expert local.

Every rank runs the same number of forwards: an exchange needs every rank's tickets (a serving engine pads an idle rank with a one-row window).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29533 -m rexl3_b200.parallel.a2a_selftest
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import sys

import numpy as np
import torch
import torch.distributed as dist


def _rows(tokens, p0, bt, dev):
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)  # noqa: E731
    pos = list(range(p0, p0 + len(tokens)))
    blocks = bt[0].tolist()
    return (i32(tokens), i32(pos), i32([blocks[p // 64] * 64 + p % 64 for p in pos]), i32([0] * len(pos)), i32([p + 1 for p in pos]), bt)


def _prefill(n, dev):
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)  # noqa: E731
    return dict(seq_ids=i32([0]), q_start=i32([0]), q_len=i32([n]), pos0=i32([0]), nseq=1, max_qlen=n)


def check(ctx, steps: int) -> dict:
    from ..models import moe
    from . import ep
    R, rank, dev = ctx.world, ctx.rank, ctx.device
    cfg = dataclasses.replace(moe.CONFIGS["test-moe"], n_experts=16, top_k=4, name="test-moe-16")
    w = moe.random_moe_weights(cfg, seed=11)
    comm = ep.make_a2a_ipc(cfg, rank, R, 256, dev, ctx.ctrl)
    shard = moe.MoEGPU(w, num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=256, device=dev,
                       experts=ep.expert_range(cfg.n_experts, rank, R), a2a=comm)
    single = moe.MoEGPU(w, num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=256, device=dev)
    rng = np.random.default_rng(100 + rank)
    prompt = rng.integers(0, cfg.vocab, size=40 + 37 * rank).tolist()      # a different length on every rank
    bt = torch.zeros(4, 4, dtype=torch.int32, device=dev)
    bt[0, :4] = torch.tensor([3, 7, 5, 9], dtype=torch.int32)
    torch.cuda.synchronize()
    dist.barrier(group=ctx.ctrl)
    equal, p0, toks = True, 0, prompt
    for s in range(steps + 1):
        kw = dict(prefill=_prefill(len(toks), dev)) if s == 0 else dict(max_ctx=256)
        got = shard.forward_rows(*_rows(toks, p0, bt, dev), **kw)[:, :cfg.vocab].clone()
        want = single.forward_rows(*_rows(toks, p0, bt, dev), **kw)[:, :cfg.vocab].clone()
        equal = equal and bool(torch.equal(got, want))
        p0 += len(toks)
        toks = [int(want[-1].argmax())]
    torch.cuda.synchronize()
    shard.check()
    flag = torch.tensor([1 if equal else 0], dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=ctx.ctrl)
    dist.barrier(group=ctx.ctrl)
    comm.g.close()
    return dict(model=cfg.name, ranks=R, forwards=steps + 1, bitwise_equal_to_one_gpu=bool(int(flag)))


def timing(ctx, rows: int, iters: int, link_gbs: float) -> dict:
    from ..models import moe
    from . import ep
    R, rank, dev, M = ctx.world, ctx.rank, ctx.device, rows
    cfg = dataclasses.replace(moe.CONFIGS["moe-spec-30b"], n_layers=2, vocab=8192, name="moe-spec-30b-2L")
    blocks = M // 64 + 2
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)  # noqa: E731
    pos = torch.arange(M, dtype=torch.int32, device=dev)
    bt = torch.zeros(2, blocks, dtype=torch.int32, device=dev)
    bt[0] = torch.arange(blocks, dtype=torch.int32, device=dev)
    slots = (bt[0][(pos // 64).long()] * 64 + pos % 64).to(torch.int32)
    ids = ((pos * (7 + rank) + 13 * rank) % cfg.vocab).to(torch.int32)
    args = (ids, pos, slots, torch.zeros(M, dtype=torch.int32, device=dev), pos + 1, bt)
    pf = dict(seq_ids=i32([0]), q_start=i32([0]), q_len=i32([M]), pos0=i32([0]), nseq=1, max_qlen=M)
    last = i32([M - 1]).long()

    def run(model):
        for _ in range(3):
            model.forward_rows(*args, prefill=pf, logit_rows=last)
        torch.cuda.synchronize()
        dist.barrier(group=ctx.ctrl)
        ts = []
        for _ in range(iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            model.forward_rows(*args, prefill=pf, logit_rows=last)
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        model.check()
        t = torch.tensor([sorted(ts)[len(ts) // 2]], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=ctx.ctrl)
        return float(t[0])

    single = moe.MoEGPU(cfg, num_pages=blocks + 1, max_rows=64, max_seqs=2, max_blocks_per_seq=blocks, max_prefill_rows=M, device=dev, seed=3)
    ms_single = run(single)
    del single
    torch.cuda.empty_cache()
    comm = ep.make_a2a_ipc(cfg, rank, R, M, dev, ctx.ctrl)
    shard = moe.MoEGPU(cfg, num_pages=blocks + 1, max_rows=64, max_seqs=2, max_blocks_per_seq=blocks, max_prefill_rows=M, device=dev, seed=3,
                       experts=ep.expert_range(cfg.n_experts, rank, R), a2a=comm)
    torch.cuda.synchronize()
    dist.barrier(group=ctx.ctrl)
    ms = run(shard)
    k, d = cfg.top_k, cfg.d_model
    out_b = M * k * (R - 1) / R * d * 2            # expected bytes a rank stores into its peers per layer (uniform routing): rows out ...
    back_b = M * k * (R - 1) / R * d * 4           # ... and f32 results stored back into the home ranks
    link_ms = (out_b + back_b) / (link_gbs * 1e9) * 1e3 * cfg.n_layers
    dist.barrier(group=ctx.ctrl)
    comm.g.close()
    return dict(model=cfg.name, ranks=R, rows_per_rank=M, ms_per_forward=round(ms, 3), tokens_per_s=round(R * M / ms * 1e3),
                one_gpu_all_experts_ms=round(ms_single, 3), one_gpu_tokens_per_s=round(M / ms_single * 1e3),
                speedup_over_one_gpu=round(R * ms_single / ms, 3), nvlink_mb_per_rank_per_layer=round((out_b + back_b) / 1e6, 1),
                nvlink_ms_per_forward_at_link_rate=round(link_ms, 3), link_gbs=link_gbs)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=7)
    ap.add_argument("--steps", type=int, default=3, help="decode steps after the prefill in the correctness part")
    ap.add_argument("--link-gbs", type=float, default=770.0, help="measured peer copy bandwidth per direction")
    ap.add_argument("--skip-timing", action="store_true")
    a = ap.parse_args()
    from . import runtime
    ctx = runtime.init(timeout_s=300)
    out = dict(bench="a2a_selftest", check=check(ctx, a.steps))
    if not a.skip_timing:
        out["timing"] = timing(ctx, a.rows, a.iters, a.link_gbs)
    if ctx.rank == 0:
        print(json.dumps(out))
    ok = out["check"]["bitwise_equal_to_one_gpu"]
    runtime.shutdown(ctx)
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
