"""Long-context serving on the 27B-class dense GQA model (EXL3 4.0 bpw, random init) with an FP8 (E4M3, per-head scales) KV cache of
64-token pages: prefill one prompt of `--prompt` tokens (default 262,144) in chunks of 8192, then decode `--decode` tokens at batch 1.

    python -m rexl3_b200.bench.long_context                          # one GPU (34 GB of FP8 KV)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29522 \
        -m rexl3_b200.bench.long_context                             # tensor parallel: every chunk's rows are split over the ranks between
                                                                     # the projections (reduce-scatter / all-gather inside the GEMM kernels)
Reports prefill seconds and tokens/s (host clock around the engine, it includes every chunk's launch and the first sampled token) and
decode tokens/s (CUDA events; under tensor parallelism the maximum over ranks).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="dense-27b")
    ap.add_argument("--prompt", type=int, default=262144)
    ap.add_argument("--chunk", type=int, default=8192)
    ap.add_argument("--decode", type=int, default=512)
    ap.add_argument("--kv-dtype", default="fp8", choices=["fp8", "bf16"])
    args = ap.parse_args()
    import numpy as np
    import torch
    import torch.distributed as dist
    from ..engine import Engine, Request
    from ..models import dense
    from ..sampling import GREEDY
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    cfg = dense.CONFIGS[args.model]
    P, D = args.prompt, args.decode
    blocks = (P + D + dense.PAGE - 1) // dense.PAGE + 2
    pages = blocks + 8
    calib = np.random.default_rng(5).integers(0, cfg.vocab, size=256).tolist()
    ctx = None
    if world > 1:
        from ..engine.tp_backend import DenseTpBackend, follow
        from ..parallel import runtime as tprt
        ctx = tprt.init(timeout_s=900)
        shard, group = tprt.build_dense_tp(ctx, cfg, num_pages=pages, max_rows=args.chunk, max_slots=2, max_blocks_per_seq=blocks, seed=0, kv_dtype=args.kv_dtype)
        shard.calibrate_kv(calib)
        if rank != 0:
            ex = follow(shard, 2, ctx.ctrl)
            t = torch.tensor([ex.marks[0].elapsed_time(ex.marks[1])], dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=ctx.ctrl)
            tprt.shutdown(ctx, group)
            return 0
        be = DenseTpBackend(shard, 2, ctx.ctrl)
    else:
        from ..engine.gpu_backend import DenseGpuBackend
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        model = dense.DenseGPU(cfg, num_pages=pages, max_rows=256, max_seqs=2, max_blocks_per_seq=blocks, max_prefill_rows=args.chunk, seed=0,
                               kv_dtype=args.kv_dtype)
        model.calibrate_kv(calib)
        be = DenseGpuBackend(model, max_slots=2)
    eng = Engine(be, None, window_rows=1, prefill_chunk=args.chunk, spec="none", prefill_policy="serial")
    prompt = np.random.default_rng(9).integers(0, cfg.vocab, size=P).tolist()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    eng.submit(Request("long", prompt, D + 4, GREEDY))
    got = 0
    while got == 0:
        for ev in eng.step():
            if ev.kind == "tokens":
                got += len(ev.tokens)
            if ev.kind == "error":
                raise SystemExit(f"prefill failed: {ev.message}")
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    for _ in range(3):
        eng.step()

    def mark():
        if world > 1:
            be.mark()
            return be.ex.marks[-1]
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e
    steps = D - 3 - 1
    e0 = mark()
    for _ in range(steps):
        eng.step()
    e1 = mark()
    if world > 1:
        be.sync_all()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        be.stop()
        t = torch.tensor([ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=ctx.ctrl)
        ms = float(t[0])
    kvb = cfg.kv_bytes_per_token(1 if args.kv_dtype == "fp8" else 2)
    print(json.dumps({"bench": "long_context", "model": cfg.name, "n_gpus": world, "parallelism": f"tp{world}", "kv_dtype": args.kv_dtype, "prompt": P,
                      "chunk": args.chunk, "prefill_s": round(prefill_s, 2), "prefill_tokens_per_s": round(P / prefill_s, 1), "decode_steps": steps,
                      "decode_tokens_per_s": round(steps / (ms / 1e3), 2), "ms_per_token": round(ms / steps, 3),
                      "kv_gb_total": round(kvb * (P + D) / 1e9, 2), "data": "synthetic", "dtype": "bf16 activations, EXL3 4.0 bpw weights"}))
    if world > 1:
        tprt.shutdown(ctx, group)
    return 0


if __name__ == "__main__":
    sys.exit(main())
