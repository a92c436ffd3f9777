#!/usr/bin/env python
"""Headline benchmark: decode tokens/s (batch 64 and batch 1) and p50 time-to-first-token at an 8192-token prompt on the
27B-class dense GQA decoder (64 layers, d_model 5120, 40q/8kv x 128, FFN 17408, vocab 151936) with random-init weights
quantized to EXL3 4.0 bpw and a paged bf16 KV cache of 64-token pages.  Synthetic uniform-random prompts.

    python bench.py --gpus N --steps K --warmup W          # this engine
    python bench.py --impl reference ...                   # the reference arm (prints why it is unavailable here)

For N > 1 the driver launches one rank per GPU with torch.distributed.run and the ONE model is sharded over the GPUs
(tensor parallelism, the same 64 sequences: strong scaling); rank 0 runs the engine, the others follow in lockstep.  Every
number is timed on the device with CUDA events recorded at the same point of every rank's stream and reduced as the MAX
over ranks.  A "step" is one decode step of the whole batch (64 tokens).  Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

PROMPT = 8192
BATCH = 64
# the reference publishes nothing on this hardware; its closest number is Qwen3.8-27B on one GB10: 62.2 tok/s, one stream,
# speculation on (docs/packs/qwen3.8-27b.md:57) - used only for the informational vs_baseline of the batch-1 figure
REFERENCE_PUBLISHED_BS1_TOK_S = 62.2


def clocks_monitor(path, gpu_index):
    q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    try:
        f = open(path, "w")
        return subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(gpu_index)],
                                stdout=f, stderr=subprocess.DEVNULL), f
    except OSError:
        return None, None


def clocks_summary(path):
    sm, mx, reasons = [], 0.0, set()
    try:
        for line in open(path):
            p = [x.strip() for x in line.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1]))
                mx = max(mx, float(p[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
    except OSError:
        pass
    busy = [x for x in sm if x > 0]
    return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm():
    print(json.dumps({"impl": "reference",
                      "unavailable": "the reference is a Rust 1.89 workspace (no setup.py/pyproject.toml; pip reports 'not installable') and "
                                     "neither cargo nor rustc exists in this image, so its public API (the rexl3-serve binary) cannot be built"}))
    return 0


def _leave(tprt, ctx, group, collective: str) -> None:
    """End of a multi-rank run.  The product path tears the group down in order.  The NCCL comparison arm created an NCCL communicator,
    whose teardown inside destroy_process_group did not return on 8 GPUs: it leaves through a last barrier on the control group and a hard
    exit instead (nothing is in flight: the device is synchronised first)."""
    if collective == "fused":
        tprt.shutdown(ctx, group)
        return
    import torch
    import torch.distributed as dist
    torch.cuda.synchronize()
    dist.barrier(group=ctx.ctrl)
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--model", default="dense-27b")
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--prompt", type=int, default=PROMPT)
    ap.add_argument("--ttft-samples", type=int, default=5)
    ap.add_argument("--collective", default="fused", choices=["fused", "nccl"],
                    help="N > 1: fused peer-memory kernels (default) or NCCL all-reduce in decode windows (the comparison baseline)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    args.warmup = max(3, args.warmup)

    import numpy as np
    import torch
    import torch.distributed as dist
    from rexl3_b200.engine import Engine, Request
    from rexl3_b200.engine.gpu_backend import DenseGpuBackend
    from rexl3_b200.models import dense
    from rexl3_b200.ops import lib as oplib
    from rexl3_b200.sampling import GREEDY

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    cfg = dense.CONFIGS[args.model]
    B, P, K, W = args.batch, args.prompt, args.steps, args.warmup
    new_tokens = 2 * (K + W) + 8
    blocks_per_seq = (P + new_tokens + dense.PAGE - 1) // dense.PAGE + 1
    pages = (B + 1) * blocks_per_seq
    need = (pages * cfg.kv_bytes_per_token() * dense.PAGE + cfg.weight_params() * cfg.bits / 8) / world + 6e9
    free, _total = torch.cuda.mem_get_info()
    if need > free:
        raise SystemExit(f"bench needs about {need / 1e9:.0f} GB on the device, {free / 1e9:.0f} GB are free")
    t0 = time.time()
    ctx = group = None
    if world > 1:
        # tensor parallelism: ONE model sharded over the GPUs, the same 64 sequences (strong scaling); rank 0 runs the engine
        from rexl3_b200.engine.tp_backend import DenseTpBackend, follow
        from rexl3_b200.parallel import runtime as tprt
        ctx = tprt.init(timeout_s=600)
        shard, group = tprt.build_dense_tp(ctx, cfg, num_pages=pages, max_rows=P, max_slots=B + 1, max_blocks_per_seq=blocks_per_seq, seed=0,
                                            collective=args.collective)
        if rank != 0:
            ex = follow(shard, B + 1, ctx.ctrl)
            m = ex.marks
            t = torch.tensor([m[0].elapsed_time(m[1]), m[2].elapsed_time(m[3])], dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=ctx.ctrl)
            _leave(tprt, ctx, group, args.collective)
            return 0
        backend = DenseTpBackend(shard, B + 1, ctx.ctrl)
        nvls = bool(getattr(group, "mm_mc_base", 0))
    else:
        model = dense.DenseGPU(cfg, num_pages=pages, max_rows=256, max_seqs=B + 1, max_blocks_per_seq=blocks_per_seq, max_prefill_rows=P, seed=rank)
        backend = DenseGpuBackend(model, max_slots=B + 1)
    engine = Engine(backend, None, window_rows=B, prefill_chunk=P, spec="none", prefill_policy="serial")
    torch.cuda.synchronize()
    build_s = time.time() - t0
    rng = np.random.default_rng(1234)
    prompts = [rng.integers(0, cfg.vocab, size=P).tolist() for _ in range(B)]

    def barrier():
        if world > 1:
            backend.sync_all()
        torch.cuda.synchronize()

    def mark():
        """A CUDA event on this rank's stream and, under tensor parallelism, at the same point of every follower's stream."""
        if world > 1:
            backend.mark()
            return backend.ex.marks[-1]
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        return ev

    # ---------------------------------------------------------------- prefill all sequences, timing TTFT through the public API
    ttfts = []
    warm = Request("warm", prompts[0][:P], 1, GREEDY)
    engine.submit(warm)
    engine.run_until_idle()          # compiles nothing, but sets kernel attributes and warms the allocator
    for i in range(B):
        barrier() if i < args.ttft_samples else None
        t = time.perf_counter()
        engine.submit(Request(f"s{i}", prompts[i], new_tokens, GREEDY))
        got = False
        while not got:
            for ev in engine.step():
                if ev.kind == "tokens" and ev.id == f"s{i}":
                    got = True
                if ev.kind == "error":
                    raise SystemExit(f"prefill failed: {ev.message}")
            if got:
                break
        torch.cuda.synchronize()
        if i < args.ttft_samples:
            ttfts.append((time.perf_counter() - t) * 1e3)
        # sequences already prefilled must not decode while the others are still reading their prompts: hold them
        engine.pause_decode = i + 1 < B
    ttft_p50 = statistics.median(ttfts)      # host clock on the rank that serves the request; it waits for every rank's shard

    # ---------------------------------------------------------------- batch-64 decode, device-timed, through the engine
    def run_steps(n):
        for _ in range(n):
            engine.step()

    run_steps(W)
    clk_path = os.path.join(tempfile.mkdtemp(prefix="rexl3_bench_"), f"clocks_rank{rank}.csv")
    mon, mon_f = clocks_monitor(clk_path, local)
    time.sleep(0.3)
    barrier()
    l0 = oplib.launch_count
    st0 = backend.stats()
    tw0 = time.perf_counter()
    e0 = mark()
    run_steps(K)
    e1 = mark()
    barrier()
    wall_ms = (time.perf_counter() - tw0) * 1e3
    dev_ms = e0.elapsed_time(e1)
    st1 = backend.stats()
    if mon is not None:
        time.sleep(0.25)
        mon.terminate()
        mon.wait()
        mon_f.close()
    # kernels replayed from captured decode graphs plus those launched eagerly inside the timed region (this rank's; every rank launches the same list)
    launches = (st1["replayed_kernels"] - st0["replayed_kernels"]) + (oplib.launch_count - l0)
    h2d = (st1["h2d_bytes"] - st0["h2d_bytes"]) / K
    d2h = (st1["d2h_bytes"] - st0["d2h_bytes"]) / K

    # ---------------------------------------------------------------- batch-1 decode: cancel all but one sequence
    for i in range(1, B):
        engine.cancel(f"s{i}")
    engine.take_events()
    run_steps(W)
    barrier()
    e2 = mark()
    run_steps(K)
    e3 = mark()
    barrier()
    bs1_ms = e2.elapsed_time(e3)
    if world > 1:
        backend.stop()
        t = torch.tensor([dev_ms, bs1_ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=ctx.ctrl)      # device time: max over ranks
        dev_ms, bs1_ms = float(t[0]), float(t[1])
    tok_s_bs64 = B * K / (dev_ms / 1e3)
    e2e_tok_s = B * K / (wall_ms / 1e3)
    tok_s_bs1 = K / (bs1_ms / 1e3)

    if rank == 0:
        clocks = clocks_summary(clk_path)
        out = {
            "metric": "decode tok/s (bs64, whole job) on 8192-token prompts; bs1 and p50 TTFT@8K in extra keys",
            "value": round(tok_s_bs64, 2), "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": round(dev_ms / K, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"model": f"{cfg.name}: {cfg.n_layers}L d{cfg.d_model} {cfg.n_q}q/{cfg.n_kv}kv x{cfg.head_dim} ffn{cfg.ffn} vocab{cfg.vocab}, "
                                f"EXL3 {cfg.bits} bpw random-init, paged bf16 KV (64-token pages)",
                       "global_batch": B, "seq_len": P, "decode_tokens_timed": K,
                       "parallelism": f"tp{world}" + ("" if world == 1 else (" (GEMM epilogue reduce-scatter and all-gather-fed GEMM for prefill, one-shot all-reduce for decode windows, "
                                                                              "all over NVLink peer memory" + (", 64-row windows summed in the switch (multimem.ld_reduce)" if nvls else "") + ", no NCCL on the step)" if args.collective == "fused" else
                                                                              " (COMPARISON RUN: NCCL all-reduce in decode windows)")),
                       "l2": "inputs larger than L2 every step (11 GB of weights + the batch's KV are streamed)"},
            "decode_tok_s_bs1": round(tok_s_bs1, 2), "ms_per_step_bs1": round(bs1_ms / K, 4),
            "ttft_p50_ms_8k": round(ttft_p50, 2), "ttft_samples": len(ttfts),
            "vs_published_gb10_bs1": round(tok_s_bs1 / REFERENCE_PUBLISHED_BS1_TOK_S, 3),
            "e2e": {"value": round(e2e_tok_s, 2), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                    "api": "rexl3_b200.engine.Engine.step (pinned-host row arrays up, candidate ids/values down, keyed sampler on the host)"},
            "gpu_launches": int(launches), "clocks": clocks, "build_s": round(build_s, 1),
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        _leave(tprt, ctx, group, args.collective)
    return 0


if __name__ == "__main__":
    sys.exit(main())
