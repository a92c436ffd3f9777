"""Batch decode on the MLA + MoE decoder (DeepSeek-V3 shape: 61 layers, d_model 7168, 128 heads, q_lora 1536, kv_lora 512, rope 64,
256 routed MXFP4 experts of FFN 2048 top-8 + shared expert, EXL3 2.0 / 2.5 bpw attention and shared weights, random init) with
expert parallelism plus head-parallel attention over N GPUs:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29521 \
        -m rexl3_b200.bench.mla_moe --batch 64 --prompt 8192 --steps 16

The full model needs about 45 GB of expert weights per GPU at 8 ranks and does not fit fewer than four GPUs; `--layers` runs a
shallower stack of the same layer shapes (reported as such).  Device time with CUDA events, rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import sys
import time


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="mla-moe-671b")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=8192)
    ap.add_argument("--chunk", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=0)
    args = ap.parse_args()
    import numpy as np
    import torch
    import torch.distributed as dist
    from ..engine import Engine, Request
    from ..engine.gpu_backend import DenseGpuBackend
    from ..engine.lockstep import LockstepLeader, follow
    from ..models import dense, mla
    from ..parallel import ep as eplib
    from ..sampling import GREEDY
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    cfg = mla.CONFIGS[args.model]
    if args.layers:
        cfg = dataclasses.replace(cfg, n_layers=args.layers, name=f"{cfg.name}[first {args.layers} layers]")
    B, P, K, W = args.batch, args.prompt, args.steps, max(3, args.warmup)
    new_tokens = K + W + 8
    blocks = (P + new_tokens + dense.PAGE - 1) // dense.PAGE + 1
    pages = (B + 1) * blocks
    ctx = comm = None
    heads = experts = None
    if world > 1:
        from ..parallel import runtime as rt
        ctx = rt.init(timeout_s=900)
        comm = eplib.make_ipc(cfg, rank, world, args.chunk, ctx.device, ctx.ctrl)
        experts = eplib.expert_range(cfg.n_experts, rank, world)
        hp = cfg.n_heads // world
        heads = (rank * hp, (rank + 1) * hp)
    else:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    t0 = time.time()
    model = mla.MlaMoEGPU(cfg, num_pages=pages, max_rows=256, max_seqs=B + 1, max_blocks_per_seq=blocks, max_prefill_rows=args.chunk, seed=0,
                          heads=heads, experts=experts, comm=comm, rank=rank)
    inner = DenseGpuBackend(model, max_slots=B + 1)
    torch.cuda.synchronize()
    build_s = time.time() - t0
    if world > 1 and rank != 0:
        follow(inner, ctx.ctrl)
        torch.cuda.synchronize()
        dist.barrier(group=ctx.ctrl)
        dist.destroy_process_group()
        return 0
    be = LockstepLeader(inner, ctx.ctrl) if world > 1 else inner
    eng = Engine(be, None, window_rows=B, prefill_chunk=args.chunk, spec="none", prefill_policy="serial")
    rng = np.random.default_rng(11)
    for i in range(B):
        eng.submit(Request(f"s{i}", rng.integers(0, cfg.vocab, size=P).tolist(), new_tokens, GREEDY))
    eng.pause_decode = True
    t0 = time.perf_counter()
    while any(s.prefilled < s.prompt_len or s.generated == 0 for s in eng.seqs.values()) or eng.waiting:
        eng.step()
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    eng.pause_decode = False
    for _ in range(W):
        eng.step()
    torch.cuda.synchronize()
    c0 = dict(eng.counters)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    tw = time.perf_counter()
    e0.record()
    for _ in range(K):
        eng.step()
    e1.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - tw
    ms = e0.elapsed_time(e1)
    toks = eng.counters["decode_tokens"] - c0["decode_tokens"]
    if world > 1:
        be.stop()
        dist.barrier(group=ctx.ctrl)
    print(json.dumps({"bench": "mla_moe", "model": cfg.name, "n_gpus": world, "parallelism": f"ep{world} + head-parallel attention" if world > 1 else "single",
                      "batch": B, "prompt": P, "steps": K, "decode_tokens_per_s": round(toks / (ms / 1e3), 2), "ms_per_step": round(ms / K, 3),
                      "e2e_tokens_per_s": round(toks / wall, 2), "prefill_s_total": round(prefill_s, 2),
                      "prefill_tokens_per_s": round(B * P / prefill_s, 1), "weight_gb_this_rank": round(model.weight_bytes() / 1e9, 2),
                      "dtype": "bf16 activations; MXFP4 experts; EXL3 2.0/2.5 bpw attention + shared", "data": "synthetic", "build_s": round(build_s, 1)}))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
