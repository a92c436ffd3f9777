"""``python -m rexl3_b200.quant`` - make an EXL3 pack: random-init weights of a built-in architecture (N(0, 0.02) from a seed), rotated
and trellis-quantized with the native Viterbi encoder, written as `config.json` + `model.safetensors`.  Counterpart of the
reference's `rexl3-quant` for the benchmark models.  Default: no calibration data (nearest trellis path per tile); `--calibrate ROWS` runs the fp32 teacher
over synthetic token sequences, accumulates every layer's input Hessian and codes with LDLQ error feedback."""
from __future__ import annotations

import argparse
import dataclasses
import sys
import time


def main(argv=None) -> int:
    from ..models import dense, hybrid
    from . import quantize
    p = argparse.ArgumentParser(prog="rexl3-quant", allow_abbrev=False)
    p.add_argument("--arch", required=True, choices=sorted([k for k, v in dense.CONFIGS.items() if type(v) is dense.DenseConfig] + list(hybrid.CONFIGS)))
    p.add_argument("--out", required=True)
    p.add_argument("--bits", type=float, default=0.0, help="override the architecture's bits per weight (1, 1.5, ... 8)")
    p.add_argument("--mtp", action="store_true", help="dense family: add one multi-token-prediction block (eh_proj + one decoder layer + its norm) to the pack")
    p.add_argument("--vision", default=None, metavar="CONFIG",
                   help="dense family: store a vision tower of this built-in shape beside the pack (vision.safetensors + vision_config; random init "
                        "from --seed, output width = the model's), for `rexl3-serve --vision-tower pack`")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--threads", type=int, default=0)
    p.add_argument("--layers", type=int, default=0, help="quantize only the first N layers (smoke runs)")
    p.add_argument("--calibrate", type=int, default=0, metavar="ROWS",
                   help="calibration rows: run the fp32 teacher over ROWS synthetic tokens (sequences of --calibrate-cols) and code with LDLQ")
    p.add_argument("--calibrate-cols", type=int, default=256)
    p.add_argument("--damp", type=float, default=0.01)
    p.add_argument("--scale-search", action="store_true", help="try a few output scales per tensor on a sample of tiles and keep the best")
    p.add_argument("--device", default="cpu", help="cpu (host Viterbi, all cores) or cuda (one CTA per tile; same bits)")
    a = p.parse_args(argv)
    is_hybrid = a.arch in hybrid.CONFIGS
    cfg = hybrid.CONFIGS[a.arch] if is_hybrid else dense.CONFIGS[a.arch]
    if a.bits:
        cfg = dataclasses.replace(cfg, bits=a.bits)
    if a.mtp:
        if is_hybrid:
            p.error("--mtp is available for the dense family")
        cfg = dataclasses.replace(cfg, mtp=True)
    if a.layers:
        cfg = dataclasses.replace(cfg, n_layers=a.layers, **({"pattern": cfg.pattern[:a.layers]} if is_hybrid else {}))
    t0 = time.time()
    if is_hybrid:
        if a.calibrate:
            p.error("--calibrate is available for the dense family")
        w = quantize.quantize_hybrid(cfg, quantize.random_fp_weights_hybrid(cfg, a.seed), seed=a.seed, threads=a.threads, device=a.device)
        quantize.write_pack(a.out, w)
        print(f"rexl3-quant: wrote {a.out} ({cfg.name}, {cfg.bits:g} bpw, {cfg.n_layers} layers, pattern {cfg.pattern}) in {time.time() - t0:.1f} s")
        return 0
    fp = quantize.random_fp_weights(cfg, a.seed)
    hessians, extra = None, None
    if a.calibrate:
        import numpy as np
        from . import teacher
        rng = np.random.default_rng(a.seed + 1)
        cols = max(1, min(a.calibrate_cols, a.calibrate))
        seqs = [rng.integers(0, cfg.vocab, size=cols).tolist() for _ in range(max(1, a.calibrate // cols))]
        hessians = teacher.capture_hessians(cfg, fp, seqs, device="cuda" if a.device != "cpu" else "cpu")
        extra = {"calibration": {"rows": len(seqs), "cols": cols, "data": "synthetic uniform tokens", "damp": a.damp}}
    w = quantize.quantize_dense(cfg, fp, seed=a.seed, threads=a.threads, device=a.device, hessians=hessians, damp=a.damp, scale_search=a.scale_search)
    quantize.write_pack(a.out, w, extra)
    if a.vision:
        import torch
        from ..vision import tower as vt
        if a.vision not in vt.CONFIGS:
            p.error(f"unknown --vision {a.vision!r}; known: {sorted(vt.CONFIGS)}")
        vt.save_tower(a.out, vt.VisionTower(dataclasses.replace(vt.CONFIGS[a.vision], out_dim=cfg.d_model), seed=a.seed, device="cpu", dtype=torch.bfloat16))
    print(f"rexl3-quant: wrote {a.out} ({cfg.name}, {cfg.bits:g} bpw, {cfg.n_layers} layers{', vision tower ' + a.vision if a.vision else ''}) "
          f"in {time.time() - t0:.1f} s")
    return 0


if __name__ == "__main__":
    sys.exit(main())
