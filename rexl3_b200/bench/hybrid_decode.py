"""Decode and prefill throughput of the hybrid (Mamba2 + NoPE GQA) decoder: 56 layers (48 Mamba2 with 128 heads x 64, state 128, 8 groups;
8 attention with 32q / 2kv x 128), d_model 4096, dense FFN 14336, vocab 131072, EXL3 4.0 bpw, random init.

    python -m rexl3_b200.bench.hybrid_decode --batch 1 16 --prompt 2048 --steps 32

For each batch size: prompts of `--prompt` tokens are prefilled through the engine (chunked), then `--steps` decode rounds are timed on
the device after warm-up rounds (CUDA-graph replay, one row per stream: this family takes no draft rows).  Reports decode tokens/s,
ms per round, prefill tokens/s (host wall clock around the prefill steps, device drained), and the resident recurrent-state bytes.
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="hybrid-h-56l")
    ap.add_argument("--batch", type=int, nargs="+", default=[1, 16])
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--prefill-chunk", type=int, default=2048)
    args = ap.parse_args()
    import numpy as np
    import torch
    from ..engine import Engine, Request
    from ..engine.gpu_backend import HybridGpuBackend
    from ..models import dense, hybrid
    from ..ops import lib as oplib
    from ..sampling import GREEDY
    cfg = hybrid.CONFIGS[args.model]
    P, K, W = args.prompt, args.steps, max(3, args.warmup)
    Bmax = max(args.batch)
    new_tokens = K + W + 8
    blocks = (P + new_tokens + dense.PAGE - 1) // dense.PAGE + 1
    model = hybrid.HybridGPU(cfg, num_pages=(Bmax + 1) * blocks, max_rows=256, max_seqs=Bmax + 1, max_blocks_per_seq=blocks,
                             max_prefill_rows=args.prefill_chunk, seed=0)
    out = []
    for B in args.batch:
        be = HybridGpuBackend(model, max_slots=Bmax + 1)
        eng = Engine(be, None, window_rows=max(B, 1), prefill_chunk=args.prefill_chunk, spec="none")
        rng = np.random.default_rng(7)
        for i in range(B):
            eng.submit(Request(f"s{i}", rng.integers(0, cfg.vocab, size=P).tolist(), new_tokens, GREEDY))
        eng.pause_decode = True
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        while any(s.prefilled < s.prompt_len or s.generated == 0 for s in eng.seqs.values()) or eng.waiting:
            for ev in eng.step():
                if ev.kind == "error":
                    raise RuntimeError(ev.message)
        torch.cuda.synchronize()
        prefill_s = time.perf_counter() - t0
        eng.pause_decode = False
        for _ in range(W):
            eng.step()
        torch.cuda.synchronize()
        c0, n0 = dict(eng.counters), oplib.launch_count + be.replayed_kernels
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            eng.step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        toks = eng.counters["decode_tokens"] - c0["decode_tokens"]
        out.append(dict(batch=B, decode_tokens_per_s=round(toks / (ms / 1e3), 2), ms_per_round=round(ms / K, 3), tokens=toks,
                        prefill_tokens_per_s=round(B * P / prefill_s, 1), prefill_s=round(prefill_s, 3),
                        kernels_per_round=(oplib.launch_count + be.replayed_kernels - n0) // K))
        del eng, be
    print(json.dumps({"bench": "hybrid_decode", "model": cfg.name, "n_gpus": 1, "prompt": P, "rounds": K, "warmup": W,
                      "dtype": "bf16 activations, fp32 recurrent state, EXL3 4.0 bpw weights", "data": "synthetic",
                      "weight_gb": round(model.weight_bytes() / 1e9, 2), "state_mb_per_stream": round(cfg.state_bytes_per_slot() / 2**20, 1),
                      "results": out}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
