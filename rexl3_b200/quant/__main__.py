"""``python -m rexl3_b200.quant`` - make an EXL3 pack: random-init weights of a built-in architecture (N(0, 0.02) from a seed), rotated
and trellis-quantized with the native Viterbi encoder, written as `config.json` + `model.safetensors`.  Counterpart of the
reference's `rexl3-quant` for the benchmark models (no calibration data is used: nearest trellis path per tile)."""
from __future__ import annotations

import argparse
import dataclasses
import sys
import time


def main(argv=None) -> int:
    from ..models import dense
    from . import quantize
    p = argparse.ArgumentParser(prog="rexl3-quant", allow_abbrev=False)
    p.add_argument("--arch", required=True, choices=sorted(k for k, v in dense.CONFIGS.items() if type(v) is dense.DenseConfig))
    p.add_argument("--out", required=True)
    p.add_argument("--bits", type=float, default=0.0, help="override the architecture's bits per weight (1, 1.5, ... 8)")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--threads", type=int, default=0)
    p.add_argument("--layers", type=int, default=0, help="quantize only the first N layers (smoke runs)")
    p.add_argument("--device", default="cpu", help="cpu (host Viterbi, all cores) or cuda (one CTA per tile; same bits)")
    a = p.parse_args(argv)
    cfg = dense.CONFIGS[a.arch]
    if a.bits:
        cfg = dataclasses.replace(cfg, bits=a.bits)
    if a.layers:
        cfg = dataclasses.replace(cfg, n_layers=a.layers)
    t0 = time.time()
    w = quantize.quantize_dense(cfg, quantize.random_fp_weights(cfg, a.seed), seed=a.seed, threads=a.threads, device=a.device)
    quantize.write_pack(a.out, w)
    print(f"rexl3-quant: wrote {a.out} ({cfg.name}, {cfg.bits:g} bpw, {cfg.n_layers} layers) in {time.time() - t0:.1f} s")
    return 0


if __name__ == "__main__":
    sys.exit(main())
