"""``python -m rexl3_b200.server`` — the serving binary (the reference's ``rexl3-serve``, crates/server/src/main.rs:3-13,
176-240): strict flags (an unknown flag is a usage error), everything CPU-side (tokenizer, template, listener) is set up
before CUDA starts, the engine runs on its own thread, a watchdog aborts a wedged process, SIGTERM drains.
"""
from __future__ import annotations

import argparse
import json
import os
import signal
import sys
import threading
import time

from ..engine import Engine, MockBackend, MockOptions
from ..sched import Admission, CacheBudget, ModelMemory, PrefixIndex
from . import api
from .http import AppState, build_app
from .runtime import EngineHandle, Metrics, RuntimeConfig
from .text import ChatFormat
from .tokenizer import load_tokenizer


def parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="rexl3-serve", allow_abbrev=False)
    p.add_argument("--model", help="pack directory (config.json, model*.safetensors, tokenizer.json ...)")
    p.add_argument("--backend", choices=["cuda", "cpu", "mock"], default="cuda")
    p.add_argument("--mock", default="", help="key=value,... options of the mock backend")
    p.add_argument("--random-init", default="", help="serve a random-init model of this built-in config instead of a pack (benchmarks)")
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=8000)
    p.add_argument("--served-model-name", default="")
    p.add_argument("--model-alias", action="append", default=[])
    p.add_argument("--slots", type=int, default=8)
    p.add_argument("--max-model-len", type=int, default=8192)
    p.add_argument("--kv-tokens", type=int, default=0, help="tokens of KV cache to reserve (0: slots * max-model-len)")
    p.add_argument("--prefill-chunk", type=int, default=4096)
    p.add_argument("--window-rows", type=int, default=64)
    p.add_argument("--kv-dtype", choices=["bf16", "fp8", "int8", "q4"], default="bf16",
                   help="fp8: E4M3 cache with per-head scales (calibrated at boot); int8: one power-of-two scale per token and KV head (no calibration); "
                        "q4: E2M1 nibbles with one E8M0 scale per 32 values (68 bytes per 128-wide row, lossy; dense family, one GPU)")
    p.add_argument("--spec", choices=["auto", "mtp", "copy", "ngram", "self", "none"], default="auto")
    p.add_argument("--intervention", metavar="DIR", default=None,
                   help="a runtime overlay directory (intervention.json + direction files): checked against the model at boot, any mismatch refuses")
    p.add_argument("--no-drafts", action="store_true")
    p.add_argument("--max-drafts", type=int, default=4)
    p.add_argument("--expert-cache-mib", type=int, default=0,
                   help="MoE packs (EXL3 experts, or MXFP4 experts under latent attention) on one GPU: keep the routed experts in a record file and page them into a device slab of this many MiB as the "
                        "router asks for them (hits, misses, bytes read and evictions are on /metrics); 0 = every expert resident")
    p.add_argument("--expert-cache-file", default=None, help="the record file (default: experts.records inside the pack; written at first start)")
    p.add_argument("--expert-cache-direct", action="store_true", help="read the record file with O_DIRECT")
    p.add_argument("--vision-tower", default=None, metavar="CONFIG",
                   help="serve image parts of chat messages through a vision tower: `pack` = the tower stored beside the pack (vision.safetensors + "
                        "vision_config), or a built-in shape with random-init weights (seed --vision-seed; its output width follows the model); "
                        "without the flag image parts are refused by name")
    p.add_argument("--vision-seed", type=int, default=0)
    p.add_argument("--vision-max-pixels", type=int, default=14 * 14 * 4 * 1280, help="pixel budget an image is resized into before it is cut into patches")
    p.add_argument("--vision-max-images", type=int, default=8, help="images one request may carry")
    p.add_argument("--spec-budget-policy", choices=["legacy", "curve", "plan", "margin", "scored"], default="legacy",
                   help="how many of a stream's drafts ride in the verify window: one acceptance rate per stream (legacy), its measured acceptance by "
                        "draft position (curve), decided before the draft (plan), trimmed again by the drafter's confidences (margin), or only the "
                        "choice of streams decided ahead and the confidences sharing the rows (scored); replies are the same under every policy")
    p.add_argument("--spec-tree", type=int, default=0, metavar="NODES",
                   help="verify draft trees of up to NODES nodes per stream (best first over the drafter's candidate lattice, the copy chain grafted in) "
                        "when the backend runs tree windows; 0 = chain windows")
    p.add_argument("--prefix-cache", choices=["on", "off"], default="on")
    p.add_argument("--prefix-cache-mib", type=int, default=4096)
    p.add_argument("--verify-pack", choices=["off", "sizes", "crc", "lock"], default="off",
                   help="check the pack before loading: file sizes against model.lock.json, per-tensor crc32.txt, or the lock's sha256 of every file")
    p.add_argument("--arbiter", action="store_true",
                   help="let the speculation arbiter decide per round how many offered drafts to verify (default: share rows by acceptance statistics)")
    p.add_argument("--state-snapshots", action="store_true",
                   help="hybrid families on CUDA: snapshot the recurrent state where a prefill slice ends so the prefix cache can serve them")
    p.add_argument("--prefix-spill-dir", default="", help="directory (e.g. on NVMe) where prefix blocks evicted from the device cache are kept and reused")
    p.add_argument("--prefix-spill-mib", type=int, default=65536)
    p.add_argument("--default-max-tokens", type=int, default=512)
    p.add_argument("--queue-depth", type=int, default=64)
    p.add_argument("--queue-timeout", type=float, default=300)
    p.add_argument("--request-timeout", type=float, default=1800)
    p.add_argument("--shutdown-grace", type=float, default=8)
    p.add_argument("--unready-after", type=int, default=3)
    p.add_argument("--exit-after", type=int, default=10)
    p.add_argument("--heartbeat-stale-secs", type=float, default=60)
    p.add_argument("--max-body-mib", type=int, default=64)
    p.add_argument("--chat-format", default=None, help="chat format id (default: from the model's config.json; see rexl3_b200.server.formats)")
    p.add_argument("--default-thinking", choices=("off", "template"), default="off",
                   help="what a chat request that names neither the thinking switch nor an effort level gets: 'off' inserts the switch set to "
                        "false where the family's switch closes the reasoning block, 'template' leaves it to the template's default")
    p.add_argument("--default-reasoning-effort", default=None, help="effort level a chat request that names none gets")
    p.add_argument("--max-rendered-prompt-mib", type=float, default=None, help="cap on a rendered prompt (default: 16 bytes per token of the window, at least 1)")
    p.add_argument("--max-json-nodes", type=int, default=300_000)
    p.add_argument("--max-json-depth", type=int, default=128)
    p.add_argument("--preparation-concurrency", type=int, default=2)
    p.add_argument("--preparation-queue", type=int, default=64)
    p.add_argument("--processing-reserve-mib", type=int, default=None, help="memory the tokenizer stage may price at once (default: derived)")
    p.add_argument("--no-graphs", action="store_true")
    p.add_argument("--device-sampler", action="store_true", help="sample and accept drafts on the GPU (verify kernel); only token ids come back")
    p.add_argument("--version", action="store_true")
    return p


def build(args):
    """-> (make_engine callable for the engine thread, tokenizer, chat format, model name, info dict).  No CUDA call happens here."""
    from ..engine.boot import BootPhases
    boot = BootPhases()
    folder = args.model if args.model and os.path.isdir(args.model) else None
    if args.backend == "mock":
        opts = MockOptions.parse(args.mock)
        opts.slots = args.slots
        vocab, name = opts.vocab, args.served_model_name or "mock"

        def make():
            be = MockBackend(opts)
            prefix = PrefixIndex(CacheBudget(args.prefix_cache_mib << 20), block_tokens=be.prefix_block_tokens()) if args.prefix_cache == "on" else None
            return Engine(be, None, window_rows=args.window_rows, prefill_chunk=args.prefill_chunk, spec="none" if args.no_drafts else args.spec,
                          max_drafts=args.max_drafts, prefix=prefix, spill=_spill_store(args, prefix), arbiter=_arbiter(args), trees=_trees(args), budget_policy=args.spec_budget_policy)
        info = {"backend": "mock"}
    else:
        from ..models import dense
        if args.random_init:
            from ..models import hybrid as hybrid_models
            from ..models import mla as mla_models
            from ..models import moe as _moe_models  # noqa: F401  (registers the MoE configs)
            if args.random_init in mla_models.CONFIGS:
                cfg = mla_models.CONFIGS[args.random_init]
            elif args.random_init in dense.CONFIGS:
                cfg = dense.CONFIGS[args.random_init]
            elif args.random_init in hybrid_models.CONFIGS:
                cfg = hybrid_models.CONFIGS[args.random_init]
            else:
                raise SystemExit(f"rexl3-serve: unknown built-in config {args.random_init!r}; known: "
                                 f"{sorted(list(dense.CONFIGS) + list(mla_models.CONFIGS) + list(hybrid_models.CONFIGS))}")
            weights = None
        else:
            if folder is None:
                raise SystemExit("rexl3-serve: --model DIR (or --random-init CONFIG) is required")
            from ..models import registry
            from ..quant import packs
            with boot.phase("scan_pack", folder=folder):
                try:
                    family, fplan = registry.probe(folder)     # architecture -> family, refusals by name, before anything is read
                except registry.FamilyError as e:
                    raise SystemExit(f"rexl3-serve: pack refused ({e.kind}): {e}")
                if not fplan.servable:
                    raise SystemExit(f"rexl3-serve: pack refused (plan_only): family `{family.id}` is known to this build for probing and memory "
                                     f"planning only ({'; '.join(fplan.notes)}); `python -m rexl3_b200.plan --pack {folder}` sizes it")
                cfg = fplan.config
            if args.verify_pack != "off":
                from ..format import verify as pack_verify
                with boot.phase("verify_pack", mode=args.verify_pack):
                    issues = (pack_verify.verify_crc(folder) if args.verify_pack == "crc"
                              else pack_verify.verify_lock(folder, sizes_only=args.verify_pack == "sizes"))
                    if issues:
                        raise SystemExit(f"rexl3-serve: pack refused by --verify-pack {args.verify_pack}: {issues[0]}"
                                         + (f" (+{len(issues) - 1} more)" if len(issues) > 1 else ""))
            with boot.phase("load_pack_host"):
                weights = packs.load_any(folder)              # header scan + refusals by name happen before CUDA starts
        vocab, name = cfg.vocab, args.served_model_name or cfg.name
        args._model_cfg = cfg
        kv_tokens = args.kv_tokens or args.slots * args.max_model_len
        info = {"backend": args.backend, "kv_pool_tokens": kv_tokens, "pack_validated": weights is not None, "boot": boot.report}
        if weights is not None:
            from ..format import verify as pack_verify
            info["pack_fingerprint"] = pack_verify.fingerprint(folder)

        world = int(os.environ.get("WORLD_SIZE", "1"))

        def make_tp():
            """Rank 0 of a tensor-parallel group (the other ranks run `follow_rank`): the engine over the lockstep TP backend."""
            from ..engine.tp_backend import DenseTpBackend
            from ..parallel import runtime as tprt
            ctx = tprt.init(timeout_s=600)
            _tp_boot_gate(args, cfg, ctx)
            if _is_expert_family(cfg):
                # expert parallel: every rank runs the whole step on replicated activations; rank 0's backend calls are replayed by the others
                from ..engine.lockstep import LockstepLeader
                be = LockstepLeader(_build_ep_backend(args, cfg, ctx, kv_tokens), ctx.ctrl)
                return Engine(be, None, window_rows=args.window_rows, prefill_chunk=args.prefill_chunk, spec="none" if args.no_drafts else args.spec,
                              max_drafts=args.max_drafts, prefix=None, cache_namespace=cache_namespace(name, cfg, info, args))
            blocks = -(-args.max_model_len // dense.PAGE) + 1
            pages = -(-kv_tokens // dense.PAGE) + args.slots
            shard, _group = tprt.build_dense_tp(ctx, cfg, num_pages=pages, max_rows=max(256, args.prefill_chunk), max_slots=args.slots,
                                                max_blocks_per_seq=blocks, weights=weights)
            be = DenseTpBackend(shard, args.slots, ctx.ctrl, use_graphs=not args.no_graphs)
            prefix = PrefixIndex(CacheBudget(args.prefix_cache_mib << 20), block_tokens=dense.PAGE) if args.prefix_cache == "on" else None
            return Engine(be, None, window_rows=args.window_rows, prefill_chunk=args.prefill_chunk, spec="none" if args.no_drafts else args.spec,
                          max_drafts=args.max_drafts, prefix=prefix, cache_namespace=cache_namespace(name, cfg, info, args), trees=_trees(args),
                          budget_policy=args.spec_budget_policy)

        def make():
            with boot.phase("engine", backend=args.backend, ranks=world):
                return make_inner()

        def make_inner():
            if args.backend == "cuda" and world > 1:
                return make_tp()
            if args.backend == "cpu":
                from ..engine.cpu_backend import CpuDenseBackend
                from ..models import hybrid as hybrid_models
                if isinstance(cfg, hybrid_models.HybridConfig):
                    from ..engine.cpu_backend import CpuHybridBackend
                    be = CpuHybridBackend(weights if weights is not None else hybrid_models.random_weights(cfg), max_slots=args.slots, max_rows=args.window_rows)
                else:
                    be = CpuDenseBackend(weights if weights is not None else dense.random_weights(cfg), max_slots=args.slots, max_rows=args.window_rows)
                adm, prefix, model = None, None, None
            else:
                import torch
                from ..engine.gpu_backend import DenseGpuBackend
                pages = -(-kv_tokens // dense.PAGE) + args.slots
                free, _ = torch.cuda.mem_get_info()
                from ..models import mla as mla_models
                from ..models import moe as moe_models
                is_mla = isinstance(cfg, mla_models.MlaConfig)
                is_moe = isinstance(cfg, moe_models.MoEConfig)
                from ..models import hybrid as hybrid_models
                is_hybrid = isinstance(cfg, hybrid_models.HybridConfig)
                if (is_mla or is_moe or is_hybrid) and args.kv_dtype != "bf16":
                    raise RuntimeError(f"--kv-dtype {args.kv_dtype} is available for the dense GQA family")
                kvb = cfg.kv_bytes_per_token() if is_mla else cfg.kv_bytes_per_token(2 if args.kv_dtype == "bf16" else 1)
                if args.kv_dtype == "int8":
                    kvb += cfg.n_layers * cfg.n_kv * 8          # one f32 scale per token, KV head and tensor
                if args.kv_dtype == "q4":                       # half a byte per value + one scale byte per 32 values
                    kvb = cfg.kv_bytes_per_token(1) // 2 + cfg.kv_bytes_per_token(1) // 32
                wbytes = int(mla_models.MlaMoEGPU.weight_bytes_estimate(cfg)) if is_mla else int(cfg.weight_params() * cfg.bits / 8)
                if is_hybrid:
                    wbytes += cfg.state_bytes_per_slot() * args.slots      # the recurrent-state pools are resident like weights
                if is_moe and not is_mla and args.expert_cache_mib:
                    # paged experts: the slab stands where the expert stacks would be
                    wbytes += (args.expert_cache_mib << 20) - int(cfg.n_layers * cfg.n_experts * 3 * cfg.d_model * cfg.expert_ffn * cfg.bits / 8)
                if is_mla and args.expert_cache_mib:
                    wbytes += (args.expert_cache_mib << 20) - int((cfg.n_layers - cfg.n_dense) * cfg.n_experts * 3 * cfg.d_model * cfg.expert_ffn * (0.5 + 1 / 32))
                mm = ModelMemory(wbytes, kvb, activation_reserve=2 << 30)
                adm = Admission(free, 1 << 30, mm, args.slots).with_max_context(args.max_model_len).with_kv_tokens(kv_tokens)
                adm.check(min(args.max_model_len, 1))     # fail closed: a plan that can never hold one token is refused at boot
                if pages * kvb * dense.PAGE > adm.capacity:
                    raise RuntimeError(f"memory plan refused: {kv_tokens} KV tokens need {pages * kvb * dense.PAGE >> 20} MiB, "
                                       f"{adm.capacity >> 20} MiB are available after weights and reserve")
                common = dict(num_pages=pages, max_rows=min(256, args.window_rows), max_seqs=args.slots,
                              max_blocks_per_seq=-(-args.max_model_len // dense.PAGE) + 1, max_prefill_rows=args.prefill_chunk)
                paging = None
                if args.expert_cache_mib:
                    if not (is_mla or is_moe):
                        raise RuntimeError("--expert-cache-mib: this model has no routed experts")
                    if weights is None:
                        raise RuntimeError("--expert-cache-mib pages the experts of a pack (--model DIR), not of a random-init config")
                    paging = dict(path=args.expert_cache_file or os.path.join(folder, "experts.records"), budget_bytes=args.expert_cache_mib << 20,
                                  direct=args.expert_cache_direct, tag=info.get("pack_fingerprint", ""))
                if is_mla:
                    model = mla_models.MlaMoEGPU(weights if weights is not None else cfg, expert_paging=paging, **common)
                elif is_moe:
                    model = moe_models.MoEGPU(weights if weights is not None else cfg, expert_paging=paging, **common)
                elif is_hybrid:
                    model = hybrid_models.HybridGPU(weights if weights is not None else cfg, **common)
                else:
                    model = dense.DenseGPU(weights if weights is not None else cfg, kv_dtype=args.kv_dtype, **common)
                if args.intervention:
                    from ..models import intervention as _iv
                    if not hasattr(model, "set_interventions"):
                        raise SystemExit(f"--intervention: the {type(model).__name__} executor has no overlay hook")
                    try:
                        model.set_interventions(_iv.load(args.intervention, n_layers=cfg.n_layers, d_model=cfg.d_model, model_name=None))
                    except (_iv.InterventionError, ValueError) as e:
                        raise SystemExit(f"--intervention refused: {e}")
                if args.kv_dtype == "fp8":
                    import numpy as np
                    model.calibrate_kv(np.random.default_rng(0).integers(0, cfg.vocab, size=min(256, args.prefill_chunk)).tolist())
                # the self-speculative drafter (first layers + shared head) is offered by families that define a draft depth
                if is_hybrid:
                    from ..engine.gpu_backend import HybridGpuBackend
                    be = HybridGpuBackend(model, max_slots=args.slots, use_graphs=not args.no_graphs, state_snapshots=args.state_snapshots)
                else:
                    # a model with a multi-token-prediction block drafts from it; else the self-speculative drafter where a draft depth is defined
                    mtp = args.spec in ("auto", "mtp") and not args.no_drafts and getattr(model, "mtp", None) is not None
                    be = DenseGpuBackend(model, max_slots=args.slots, use_graphs=not args.no_graphs, mtp_draft=mtp,
                                         self_draft=not mtp and args.spec in ("auto", "self") and not args.no_drafts and getattr(cfg, "draft_layers", 0) > 0)
                prefix = PrefixIndex(CacheBudget(args.prefix_cache_mib << 20), block_tokens=dense.PAGE) if args.prefix_cache == "on" else None
            return Engine(be, adm, window_rows=args.window_rows, prefill_chunk=args.prefill_chunk, spec="none" if args.no_drafts else args.spec,
                          max_drafts=args.max_drafts, prefix=prefix, cache_namespace=cache_namespace(name, cfg, info, args, model), device_sampler=args.device_sampler,
                          spill=_spill_store(args, prefix), arbiter=_arbiter(args), trees=_trees(args), budget_policy=args.spec_budget_policy)
    tok = load_tokenizer(folder, vocab)
    from . import formats
    try:
        fmt = formats.open_format(folder, getattr(args, "chat_format", None))
    except formats.FormatRefused as e:
        raise SystemExit(f"rexl3-serve: {e}")
    info["chat_format"] = fmt.id
    info["reasoning"] = fmt.caps.describe()
    return make, tok, fmt, name, info


def cache_namespace(name: str, cfg, info: dict, args, model=None) -> bytes:
    """Namespace of the prefix cache and of the spill directory: everything that decides what a KV page of some token chain holds.
    The served name alone is not enough (a re-quantised or fine-tuned pack under the same name, or an FP8 cache with newly calibrated
    per-head scales, would hash to the same chains and stale pages would be adopted at start): the pack fingerprint (for random-init
    weights the configuration and its seed), the KV dtype and a digest of the FP8 scale tensor are folded in."""
    import dataclasses
    import hashlib
    h = hashlib.sha256()
    h.update(name.encode())
    fp = info.get("pack_fingerprint")
    if fp:
        h.update(b"pack:" + str(fp).encode())
    else:
        desc = dataclasses.asdict(cfg) if dataclasses.is_dataclass(cfg) else {"name": getattr(cfg, "name", "")}
        h.update(b"random-init:" + repr(sorted(desc.items())).encode() + b":seed0")
    h.update(b"kv:" + str(getattr(args, "kv_dtype", "bf16")).encode())
    scale = getattr(model, "kv_scale", None) if model is not None else None
    if scale is not None:
        h.update(b"kv_scale:" + scale.detach().float().cpu().numpy().tobytes())
    return h.hexdigest()[:32].encode()


def _tp_boot_gate(args, cfg, ctx) -> None:
    """Every rank of the group must be about to run the same thing (raises BootGateError on all ranks otherwise)."""
    from ..models import hybrid as hybrid_models
    if isinstance(cfg, hybrid_models.HybridConfig):
        raise RuntimeError("the hybrid (Mamba2 / delta-net) family runs on one GPU per replica: start one process per GPU behind the router instead")
    from ..parallel import bootgate
    flags = dict(slots=args.slots, max_model_len=args.max_model_len, prefill_chunk=args.prefill_chunk, kv_tokens=args.kv_tokens,
                 graphs=not args.no_graphs, random_init=args.random_init or "")
    bootgate.gate(bootgate.collect_facts(cfg, world=ctx.world, pack=args.model or None, flags=flags), ctx.ctrl)


def _build_ep_backend(args, cfg, ctx, kv_tokens):
    """This rank's share of an expert-parallel group for the MoE and MLA + MoE families (experts owned by rank, MLA heads split by rank,
    activations replicated; the combine is the fused all-reduce over the symmetric arena) behind the single-GPU backend class.  The same
    construction the family benchmarks use (`bench/spec_moe.py`, `bench/mla_moe.py`)."""
    from ..engine.gpu_backend import DenseGpuBackend
    from ..models import dense
    from ..models import mla as mla_models
    from ..models import moe as moe_models
    from ..parallel import ep as eplib
    comm = eplib.make_ipc(cfg, ctx.rank, ctx.world, args.prefill_chunk, ctx.device, ctx.ctrl)
    experts = eplib.expert_range(cfg.n_experts, ctx.rank, ctx.world)
    common = dict(num_pages=-(-kv_tokens // dense.PAGE) + args.slots, max_rows=min(256, args.window_rows), max_seqs=args.slots,
                  max_blocks_per_seq=-(-args.max_model_len // dense.PAGE) + 1, max_prefill_rows=args.prefill_chunk, seed=0)
    if isinstance(cfg, mla_models.MlaConfig):
        if cfg.n_heads % ctx.world:
            raise RuntimeError(f"{cfg.n_heads} MLA heads do not split over {ctx.world} ranks")
        hp = cfg.n_heads // ctx.world
        model = mla_models.MlaMoEGPU(cfg, heads=(ctx.rank * hp, (ctx.rank + 1) * hp), experts=experts, comm=comm, rank=ctx.rank, **common)
    else:
        model = moe_models.MoEGPU(cfg, experts=experts, ep=comm, **common)
    return DenseGpuBackend(model, max_slots=args.slots, use_graphs=not args.no_graphs)


def _is_expert_family(cfg) -> bool:
    from ..models import mla as mla_models
    from ..models import moe as moe_models
    return isinstance(cfg, (mla_models.MlaConfig, moe_models.MoEConfig))


def _trees(args):
    if getattr(args, "spec_tree", 0) <= 0 or args.no_drafts:
        return None
    from ..engine import TreeConfig
    return TreeConfig(max_nodes=min(63, args.spec_tree))


def _vision(args, tok, fmt, info):
    """The image path of the chat route (server.media.VisionIngress), or None.  Refusals come at start-up, by name."""
    if not getattr(args, "vision_tower", None):
        return None
    import dataclasses
    from ..vision import tower as vt
    from .media import VisionIngress
    from_pack = args.vision_tower == "pack"
    folder = args.model if args.model and os.path.isdir(args.model) else None
    if from_pack:
        try:
            vcfg = vt.config_from_pack(folder) if folder else None
        except ValueError as e:
            raise SystemExit(f"rexl3-serve: --vision-tower pack: {e}")
        if vcfg is None:
            raise SystemExit("rexl3-serve: --vision-tower pack: the pack (--model DIR) holds no vision tower (vision.safetensors + vision_config)")
    elif args.vision_tower not in vt.CONFIGS:
        raise SystemExit(f"rexl3-serve: unknown --vision-tower {args.vision_tower!r}; known: pack, {', '.join(sorted(vt.CONFIGS))}")
    else:
        vcfg = vt.CONFIGS[args.vision_tower]
    cfg = getattr(args, "_model_cfg", None)
    if cfg is not None:
        if not hasattr(cfg, "d_model") or type(cfg).__name__ not in ("DenseConfig", "MoEConfig"):
            raise SystemExit(f"rexl3-serve: --vision-tower: the `{cfg.name}` executor takes no image rows (dense and MoE GQA decoders do)")
        if getattr(args, "spec", "") == "mtp" or int(os.environ.get("WORLD_SIZE", "1")) > 1:
            raise SystemExit("rexl3-serve: --vision-tower runs on one rank and without --spec mtp")
        if from_pack and vcfg.out_dim != cfg.d_model:
            raise SystemExit(f"rexl3-serve: --vision-tower pack: the tower writes rows of width {vcfg.out_dim}, the model is {cfg.d_model} wide")
        vcfg = dataclasses.replace(vcfg, out_dim=cfg.d_model)
    placeholder = getattr(fmt, "image_placeholder", "<|vision_start|><|image_pad|><|vision_end|>")
    tid = tok.special_id("<|image_pad|>")
    if tid is None:
        raise SystemExit("rexl3-serve: --vision-tower: the tokenizer has no <|image_pad|> token")
    fmt.serves_images = True
    cuda = args.backend == "cuda"

    def make_tower():
        import torch
        dev, dt = ("cuda", torch.bfloat16) if cuda else ("cpu", torch.float32)
        return vt.load_tower(folder, dev, dt) if from_pack else vt.VisionTower(vcfg, seed=args.vision_seed, device=dev, dtype=dt)
    info["vision"] = {"tower": vcfg.name, "out_dim": vcfg.out_dim, "patch": vcfg.patch, "merge": vcfg.merge,
                      "weights": "vision.safetensors of the pack" if from_pack else f"random init, seed {args.vision_seed}"}
    return VisionIngress(vcfg, make_tower, tid, placeholder, mrope=getattr(cfg, "mrope_sections", None) is not None, max_pixels=args.vision_max_pixels,
                         max_images=args.vision_max_images)


def _arbiter(args):
    if not args.arbiter or args.no_drafts or args.spec == "none":
        return None
    from ..spec import Arbiter
    # a window's time grows slowly with its rows (weights are read once per window): a flat cost plus a small slope per row
    return Arbiter(verify_ms=lambda streams, rows: 10.0 + 0.05 * rows)


def _spill_store(args, prefix):
    if prefix is None or not args.prefix_spill_dir:
        return None
    from ..sched.spill import SpillStore
    return SpillStore(args.prefix_spill_dir, args.prefix_spill_mib << 20)


def follow_rank(args) -> int:
    """Ranks 1.. of a tensor-parallel group: no HTTP, no scheduler - repeat the leader's launches until it stops.
    Exit status 0 on a clean stop, 70 when the group is lost or the device reports an error (the supervisor restarts the group)."""
    from ..engine.tp_backend import follow
    from ..models import dense
    from ..parallel import runtime as tprt
    try:
        if args.random_init:
            from ..models import mla as mla_models
            from ..models import moe as _moe_models  # noqa: F401  (registers the MoE configs)
            from ..models import hybrid as hybrid_models
            cfg = (mla_models.CONFIGS.get(args.random_init) or hybrid_models.CONFIGS.get(args.random_init) or dense.CONFIGS[args.random_init])
            weights = None
        else:
            from ..quant import quantize
            cfg, weights = quantize.config_from_pack(args.model), quantize.load_pack(args.model)
        kv_tokens = args.kv_tokens or args.slots * args.max_model_len
        ctx = tprt.init(timeout_s=600)
        try:
            _tp_boot_gate(args, cfg, ctx)
        except Exception as e:  # a group that disagrees is refused (exit status 2: the supervisor does not restart a refusal blindly)
            print(f"rexl3 level=error event=boot_refused rank={os.environ.get('RANK')} error={e}", file=sys.stderr, flush=True)
            return 2
        if _is_expert_family(cfg):
            import torch
            from ..engine import lockstep
            lockstep.follow(_build_ep_backend(args, cfg, ctx, kv_tokens), ctx.ctrl)
            torch.cuda.synchronize()
            return 0
        shard, group = tprt.build_dense_tp(ctx, cfg, num_pages=-(-kv_tokens // dense.PAGE) + args.slots, max_rows=max(256, args.prefill_chunk),
                                           max_slots=args.slots, max_blocks_per_seq=-(-args.max_model_len // dense.PAGE) + 1, weights=weights)
        follow(shard, args.slots, ctx.ctrl, use_graphs=not args.no_graphs)
        return 0
    except Exception as e:  # a lost leader surfaces as a transport error or a device status
        print(f"rexl3 level=error event=follower_lost rank={os.environ.get('RANK')} error={e!r}", file=sys.stderr, flush=True)
        return 70


def make_app(args, metrics: Metrics | None = None):
    make, tok, fmt, name, info = build(args)
    rc = RuntimeConfig(queue_depth=args.queue_depth, queue_timeout_s=args.queue_timeout, request_timeout_s=args.request_timeout,
                       unready_after=args.unready_after, exit_after=args.exit_after, shutdown_grace_s=args.shutdown_grace)
    handle = EngineHandle(make, rc, metrics)
    defaults = api.GenDefaults()
    if args.model and os.path.exists(os.path.join(args.model, "generation_config.json")):
        defaults = api.GenDefaults.from_dict(json.load(open(os.path.join(args.model, "generation_config.json"))))
    from . import budget, formats
    limits = budget.Limits.for_window(args.max_model_len)
    limits.body_bytes = args.max_body_mib << 20
    limits.json_nodes, limits.json_depth = args.max_json_nodes, args.max_json_depth
    limits.preparation_concurrency, limits.preparation_queue = args.preparation_concurrency, args.preparation_queue
    if args.max_rendered_prompt_mib is not None:
        limits.rendered_bytes = int(args.max_rendered_prompt_mib * (1 << 20))
    limits.processing_reserve_bytes = (args.processing_reserve_mib << 20) if args.processing_reserve_mib is not None else limits.derived_reserve()
    if args.processing_reserve_mib is None:
        raw = max(min(limits.body_bytes, limits.total_bytes) * 16, limits.json_nodes * 128) * limits.preparation_concurrency
        limits.processing_reserve_bytes = max(limits.processing_reserve_bytes, raw)
    try:
        limits.validate()
    except ValueError as e:
        raise SystemExit(f"rexl3-serve: {e}")
    if args.default_reasoning_effort is not None:
        caps = fmt.caps
        ok = caps.reasons and (caps.level(args.default_reasoning_effort) is not None
                               or (caps.effort_var and args.default_reasoning_effort in (caps.extra_vars.get(caps.effort_var) or [])))
        if not ok:
            raise SystemExit(f"rexl3-serve: --default-reasoning-effort {args.default_reasoning_effort}: this model takes "
                             f"{', '.join(caps.level_names()) or 'no effort levels'}")
    st = AppState(handle, tok, fmt, name, args.max_model_len, args.model_alias, defaults, args.default_max_tokens,
                  fingerprint=f"rexl3-b200-{name}", max_body_bytes=args.max_body_mib << 20, info=info, limits=limits,
                  default_thinking=args.default_thinking, default_effort=args.default_reasoning_effort, vision=_vision(args, tok, fmt, info))
    return build_app(st), handle


def main(argv=None) -> int:
    args = parser().parse_args(argv)
    if args.version:
        from .. import __version__
        print(f"rexl3-serve (rexl3_b200) {__version__}")
        return 0
    if args.backend == "cuda" and int(os.environ.get("WORLD_SIZE", "1")) > 1 and int(os.environ.get("RANK", "0")) != 0:
        return follow_rank(args)
    import uvicorn
    print(f"rexl3 event=start backend={args.backend} host={args.host} port={args.port}", file=sys.stderr, flush=True)
    app, handle = make_app(args)

    def watchdog():
        while True:
            time.sleep(0.25)
            if handle.wedged(args.heartbeat_stale_secs):
                print("rexl3 level=error event=wedged action=abort", file=sys.stderr, flush=True)
                os.abort()
            if handle.state == "failed":
                print(f"rexl3 level=error event=engine_failed error={handle.error!r}", file=sys.stderr, flush=True)
                os._exit(70)
    threading.Thread(target=watchdog, daemon=True).start()
    server = uvicorn.Server(uvicorn.Config(app, host=args.host, port=args.port, log_level="warning", timeout_graceful_shutdown=int(args.shutdown_grace)))

    def on_signal(signum, frame):
        print("rexl3 event=drain", file=sys.stderr, flush=True)
        handle.drain()
        server.should_exit = True
    signal.signal(signal.SIGTERM, on_signal)
    signal.signal(signal.SIGINT, on_signal)
    server.run()
    handle.stop()
    be = getattr(getattr(handle, "engine", None), "backend", None)
    if hasattr(be, "stop"):          # a tensor-parallel leader releases its followers (they exit 0 on the stop message)
        try:
            be.stop()
        except Exception:
            pass
    return 0


if __name__ == "__main__":
    sys.exit(main())
