"""Speculative decode on the MoE GQA decoder (48 layers, d_model 2048, 32q/4kv x 128, 128 experts of FFN 768, top-8, vocab 151936,
EXL3 3.0 bpw, random init): self-speculative draft (first 4 layers + shared head, chain of k = 4), one batched verify forward.

    python -m rexl3_b200.bench.spec_moe --batch 16 --steps 32
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29520 \
        -m rexl3_b200.bench.spec_moe --batch 16 --steps 32            # expert parallel, 16 experts per GPU

Reports, for speculation off and on: decode tokens/s (device time, max over ranks under expert parallelism), the mean verify-step
latency (the target forward of the window, host-timed around the backend call including its small device->host read), drafts
proposed/accepted.  With plain random weights the draft almost never matches the target, so that "on" figure shows the cost side of
speculation.  `--tail-scale 1.0 0.1 0.03` adds runs in which the layers above the draft depth write less into the residual stream, which
raises the agreement between the 4-layer draft and the target; acceptance always comes from the engine's counters, nothing is assumed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="moe-spec-30b")
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--prompt", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--drafts", type=int, default=4)
    ap.add_argument("--tail-scale", type=float, nargs="*", default=[1.0],
                    help="one run per value: the output scales of o_proj / down_proj in the layers above the draft depth are multiplied by it "
                         "(1.0 = plain random init, acceptance ~0; small values make the 4-layer draft agree with the target more often)")
    ap.add_argument("--mtp", action="store_true",
                    help="one GPU, a dense config (--model dense-27b): drafts come from a multi-token-prediction block (random init, so nothing is "
                         "accepted: the run shows what the block's lagged rows and a chain of k drafts cost per round)")
    ap.add_argument("--tree", type=int, default=0, metavar="NODES",
                    help="one GPU, self draft: a third run whose verify windows are draft trees of up to NODES nodes per stream, searched best "
                         "first over the four candidates the draft chain gives per level")
    args = ap.parse_args()
    import dataclasses
    import numpy as np
    import torch
    import torch.distributed as dist
    from ..engine import Engine, Request
    from ..engine.gpu_backend import DenseGpuBackend
    from ..engine.lockstep import LockstepLeader, follow
    from ..models import dense, moe
    from ..parallel import ep as eplib
    from ..sampling import GREEDY
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    cfg = dataclasses.replace(dense.CONFIGS[args.model], mtp=True, name=args.model + "-mtp") if args.mtp else moe.CONFIGS[args.model]
    drafter = "mtp" if args.mtp else "self"
    B, P, K, W, D = args.batch, args.prompt, args.steps, max(3, args.warmup), args.drafts
    new_tokens = (K + W) * (D + 1) * 2 + 16
    blocks = (P + new_tokens + dense.PAGE - 1) // dense.PAGE + 1
    pages = (B + 1) * blocks + 2 * B * args.tree          # a tree node outside the first chain holds up to two private pages for a round
    ctx = comm = None
    if world > 1:
        from ..parallel import runtime as rt
        ctx = rt.init(timeout_s=600)
        comm = eplib.make_ipc(cfg, rank, world, P, ctx.device, ctx.ctrl)
        experts = eplib.expert_range(cfg.n_experts, rank, world)
    else:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        experts = None

    def measure(eps: float) -> dict:
        results = {}
        for mode in ("none", drafter) + (("tree",) if args.tree > 0 and not args.mtp and world == 1 else ()):
            measure_mode(eps, mode, results)
        return results

    def measure_mode(eps: float, mode: str, results: dict) -> None:
        if args.mtp:
            model = dense.DenseGPU(cfg, num_pages=pages, max_rows=256, max_seqs=B + 1, max_blocks_per_seq=blocks, max_prefill_rows=P, seed=0)
        else:
            model = moe.MoEGPU(cfg, num_pages=pages, max_rows=256, max_seqs=B + 1, max_blocks_per_seq=blocks, max_prefill_rows=P, seed=0,
                               experts=experts, ep=comm)
            if eps != 1.0:
                model.scale_tail(cfg.draft_layers, eps)
        inner = DenseGpuBackend(model, max_slots=B + 1, self_draft=(mode in ("self", "tree")), mtp_draft=(mode == "mtp"))
        if world > 1 and rank != 0:
            follow(inner, ctx.ctrl)
            torch.cuda.synchronize()
            del model, inner
            torch.cuda.empty_cache()
            return
        be = LockstepLeader(inner, ctx.ctrl) if world > 1 else inner
        if mode == "tree":
            from ..engine import TreeConfig
            eng = Engine(be, None, window_rows=min(256, B * (args.tree + 1)), prefill_chunk=P, spec="self", max_drafts=D, prefill_policy="serial",
                         trees=TreeConfig(max_nodes=args.tree))
        else:
            eng = Engine(be, None, window_rows=B * (D + 1), prefill_chunk=P, spec=mode, max_drafts=D, prefill_policy="serial")
        rng = np.random.default_rng(7)
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
        c0, v0 = dict(eng.counters), eng.phase_ns["verify"]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            eng.step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        c1 = eng.counters
        toks = c1["decode_tokens"] - c0["decode_tokens"]
        drafted, accepted = c1["drafted"] - c0["drafted"], c1["accepted"] - c0["accepted"]
        results[mode] = dict(tokens_per_s=round(toks / (ms / 1e3), 2), ms_per_round=round(ms / K, 3), tokens=toks,
                             verify_step_ms=round((eng.phase_ns["verify"] - v0) / K / 1e6, 3), drafted=drafted, accepted=accepted,
                             acceptance=round(accepted / drafted, 4) if drafted else None, rows_per_round=(c1["rows"] - c0["rows"]) / K,
                             prefill_s=round(prefill_s, 2), **({"backend": inner.stats()} if mode == "tree" else {}))
        if world > 1:
            be.stop()
        del eng, be, inner, model
        torch.cuda.empty_cache()
    runs = [(eps, measure(eps)) for eps in args.tail_scale]
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier(group=ctx.ctrl)
    if rank == 0:
        print(json.dumps({"bench": "spec_moe", "model": cfg.name, "n_gpus": world, "parallelism": f"ep{world}" if world > 1 else "single",
                          "batch": B, "prompt": P, "rounds": K,
                          "draft": f"mtp block, chain k={D}" if args.mtp else f"self: first {cfg.draft_layers} layers + shared head, chain k={D}",
                          "dtype": f"bf16 activations, EXL3 {cfg.bits} bpw weights", "data": "synthetic (random init; tail_scale multiplies the output scales of o_proj / down_proj above the draft depth)",
                          "runs": [dict(tail_scale=eps, spec_off=r["none"], spec_on=r[drafter],
                                        speedup=round(r[drafter]["tokens_per_s"] / r["none"]["tokens_per_s"], 3),
                                        **({"spec_tree": r["tree"], "tree_nodes": args.tree,
                                            "tree_speedup": round(r["tree"]["tokens_per_s"] / r["none"]["tokens_per_s"], 3)} if "tree" in r else {}))
                                   for eps, r in runs]}))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
