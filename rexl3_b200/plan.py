"""Memory plan of a model on B200s, before anything is loaded: weight bytes, KV bytes per token, recurrent-state bytes per stream, and
what fits (KV tokens, or the longest context at a slot count) on GPUs of a given size.  The "probe / plan only" path a family needs
before it has an executor (the reference's memory model + startup plan; its `mimo` family stops there), and the same arithmetic the
server's admission uses at boot.

    python -m rexl3_b200.plan --config dense-27b --slots 64 --max-model-len 8704
    python -m rexl3_b200.plan --config mla-moe-671b --gpus 8 --slots 64 --max-model-len 8704
    python -m rexl3_b200.plan --pack /models/pack --kv-dtype fp8 --slots 32 --max-model-len 32768
"""
from __future__ import annotations

import json
import sys

GPU_BYTES = 183_359 * (1 << 20)         # what a B200 reports (MiB)
RESERVE_BYTES = 3 << 30                 # activations, scratch and allocator slack kept free on every GPU


def describe(cfg, kv_dtype: str = "bf16") -> dict:
    """Family-independent sizes of a config object of any built-in family."""
    from .models import hybrid as hy
    from .models import mla as ml
    from .models import moe as mo
    out = {"model": getattr(cfg, "name", "?"), "layers": cfg.n_layers, "d_model": cfg.d_model, "vocab": cfg.vocab}
    if isinstance(cfg, ml.MlaConfig):
        out.update(family="mla_moe", weight_bytes=int(ml.MlaMoEGPU.weight_bytes_estimate(cfg)), kv_bytes_per_token=int(cfg.kv_bytes_per_token()),
                   state_bytes_per_slot=0, shards="experts by rank, heads by rank")
    elif isinstance(cfg, hy.HybridConfig):
        out.update(family="hybrid", weight_bytes=int(cfg.weight_params() * cfg.bits / 8) + cfg.vocab * cfg.d_model * 2,
                   kv_bytes_per_token=int(cfg.kv_bytes_per_token(2 if kv_dtype == "bf16" else 1)), state_bytes_per_slot=int(cfg.state_bytes_per_slot()),
                   pattern=cfg.pattern, shards="one GPU per replica")
    elif isinstance(cfg, mo.MoEConfig):
        out.update(family="moe_gqa", weight_bytes=int(cfg.weight_params() * cfg.bits / 8) + cfg.vocab * cfg.d_model * 2,
                   kv_bytes_per_token=int(cfg.kv_bytes_per_token(2)), state_bytes_per_slot=0, shards="experts by rank")
    else:
        kvb = cfg.kv_bytes_per_token(1) // 2 + cfg.kv_bytes_per_token(1) // 32 if kv_dtype == "q4" else cfg.kv_bytes_per_token(2 if kv_dtype == "bf16" else 1)
        out.update(family="dense_gqa", weight_bytes=int(cfg.weight_params() * cfg.bits / 8) + cfg.vocab * cfg.d_model * 2,
                   kv_bytes_per_token=int(kvb), state_bytes_per_slot=0,
                   shards="columns / rows and KV heads by rank")
    return out


def plan(cfg, *, gpus: int = 1, slots: int = 16, max_model_len: int = 8192, kv_dtype: str = "bf16", gpu_bytes: int = GPU_BYTES,
         reserve_bytes: int = 3 << 30) -> dict:
    """Per-GPU budget: weights and KV split over `gpus` (replicated parts are counted as split: an optimistic bound the boot-time admission
    then checks against the real allocations), state and reserve per GPU."""
    d = describe(cfg, kv_dtype)
    w = d["weight_bytes"] // gpus
    kv = max(1, d["kv_bytes_per_token"] // gpus)
    state = d["state_bytes_per_slot"] * slots
    free = gpu_bytes - reserve_bytes - w - state
    want_tokens = slots * max_model_len
    fit_tokens = max(0, free // kv)
    d.update(gpus=gpus, slots=slots, max_model_len=max_model_len, kv_dtype=kv_dtype, per_gpu={"weights": w, "recurrent_state": state, "reserve": reserve_bytes,
             "kv_for_all_slots": want_tokens * kv, "free_after_weights_and_state": free},
             kv_tokens_that_fit=int(fit_tokens), longest_context_at_these_slots=int(fit_tokens // max(1, slots)),
             fits=bool(free > 0 and fit_tokens >= want_tokens))
    return d


def find_config(name: str):
    from .models import dense, hybrid, mla
    from .models import moe as _moe  # noqa: F401  (registers the MoE configs)
    for table in (mla.CONFIGS, hybrid.CONFIGS, dense.CONFIGS):
        if name in table:
            return table[name]
    raise KeyError(name)


def main(argv=None) -> int:
    import argparse
    p = argparse.ArgumentParser(prog="rexl3-plan", allow_abbrev=False)
    g = p.add_mutually_exclusive_group(required=True)
    g.add_argument("--config", help="a built-in architecture name")
    g.add_argument("--pack", help="a pack directory (its config.json is read; no tensor is)")
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--slots", type=int, default=16)
    p.add_argument("--max-model-len", type=int, default=8192)
    p.add_argument("--kv-dtype", choices=["bf16", "fp8", "int8", "q4"], default="bf16")
    a = p.parse_args(argv)
    try:
        if a.config:
            cfg = find_config(a.config)
        else:
            from .models import registry
            from .quant import quantize
            try:
                fam, fplan = registry.probe(a.pack)
            except registry.FamilyError as e:
                print(f"rexl3-plan: pack refused ({e.kind}): {e}", file=sys.stderr)
                return 2
            if not fplan.servable:
                # a family this build only probes: its own memory model, sized against the GPUs asked for
                m = dict(fplan.memory)
                kv = m["kv_bytes_per_token"] // (2 if a.kv_dtype != "bf16" else 1) * a.max_model_len * a.slots
                per = (m["weight_bytes"] + kv) // a.gpus + RESERVE_BYTES
                doc = dict(family=fam.id, servable=False, notes=fplan.notes, config=fplan.config, memory=m, gpus=a.gpus, slots=a.slots,
                           max_model_len=a.max_model_len, per_gpu_bytes=int(per), fits=bool(per <= GPU_BYTES))
                print(json.dumps(doc, indent=1))
                return 0 if doc["fits"] else 1
            cfg = quantize.config_from_pack(a.pack)
    except (KeyError, OSError, ValueError) as e:
        print(f"rexl3-plan: {e}", file=sys.stderr)
        return 2
    out = plan(cfg, gpus=a.gpus, slots=a.slots, max_model_len=a.max_model_len, kv_dtype=a.kv_dtype)
    print(json.dumps(out, indent=1))
    return 0 if out["fits"] else 1


if __name__ == "__main__":
    sys.exit(main())
