"""Which bits a tensor-parallel cut keeps, as data: per (matrix, rank count) the split plan of the whole matrix, the plan a rank's slice would
get by itself, and the verdict (the family-neutral half of reference crates/model/src/shard.rs:1-16).

An output column of an EXL3 GEMM accumulates over K alone, in the order fixed by the K-split count the launch is given.  A COLUMN cut
(q | k | v, gate | up, the head) keeps every column's bits exactly when the slice is launched with the WHOLE matrix's split count: `same_plan`
says the planner would pick that count for the slice anyway, `pinned` says the shard must pass the whole matrix's count (the launchers take the
count as an argument, so pinning costs nothing but the planner's choice).  A ROW cut (o_proj, down_proj) splits K across ranks: the ranks'
partial rows are summed in rank order, which is a fixed order but not the one-GPU order, so those outputs are `rank_order` - deterministic for
a rank count, not comparable bit for bit across rank counts.  `compare_slices` holds the column verdicts against the kernel on a device."""
from __future__ import annotations

from dataclasses import dataclass

from ..format import tp as tpfmt


@dataclass(frozen=True)
class ShapeProof:
    name: str
    cut: str                 # "columns" | "rows"
    K: int
    N: int
    ranks: int
    local: tuple             # (K_local, N_local) of rank 0's slice
    whole_splits: int
    local_splits: int
    verdict: str             # "same_plan" | "pinned" | "rank_order"


def plan_splits(K: int, N: int, decode_class: bool = True) -> int:
    """Mirror of the library's planner (rx_exl3_plan_splits): prefill-class launches never split K; a window splits K until strips x splits
    covers two CTAs per SM, at most half the 128-wide K chunks and at most 32."""
    if not decode_class:
        return 1
    strips, chunks = N // 128, K // 128
    return max(1, min(32, chunks // 2, (2 * 148) // max(1, strips)))


def proof_table(shapes: dict, ranks: int, decode_class: bool = True) -> list:
    """shapes: name -> (K, N, cut).  One ShapeProof per matrix for `ranks` ranks (the widest rank's slice decides)."""
    out = []
    for name, (K, N, cut) in shapes.items():
        whole = plan_splits(K, N, decode_class)
        if cut == "columns":
            n_loc = max(tpfmt.split_width(N, r, ranks).width for r in range(ranks))
            loc = plan_splits(K, n_loc, decode_class)
            out.append(ShapeProof(name, cut, K, N, ranks, (K, n_loc), whole, loc, "same_plan" if loc == whole else "pinned"))
        elif cut == "rows":
            k_loc = max(tpfmt.split_width(K, r, ranks).width for r in range(ranks))
            out.append(ShapeProof(name, cut, K, N, ranks, (k_loc, N), whole, plan_splits(k_loc, N, decode_class), "rank_order"))
        else:
            raise ValueError(f"{name}: cut must be 'columns' or 'rows', got {cut!r}")
    return out


def dense_shapes(cfg) -> dict:
    """The dense GQA family's cuts (models/dense_tp.py): q | k | v, gate | up and the head by columns; o_proj and down_proj by rows."""
    return dict(qkv=(cfg.d_model, cfg.qkv_width, "columns"), o=(cfg.n_q * cfg.head_dim, cfg.d_model, "rows"),
                gate_up=(cfg.d_model, 2 * cfg.ffn_padded, "columns"), down=(cfg.ffn_padded, cfg.d_model, "rows"),
                lm_head=(cfg.d_model, cfg.vocab_padded, "columns"))


def compare_slices(w, ranks: int, rows: int = 5, seed: int = 0) -> dict:
    """Device harness for one column-cut matrix `w` (ops.kernels.Exl3Weight): every rank's column slice, launched with the whole matrix's split
    count, must reproduce the whole launch's partial sums of its columns byte for byte.  -> {rank: True / False}."""
    import torch
    from ..ops import kernels as K
    g = torch.Generator(device=w.trellis.device).manual_seed(seed)
    x = (torch.randn(rows, w.K, device=w.trellis.device, generator=g) * 0.5).to(torch.float16)
    s = K.plan_splits(w.K, w.N, True)
    status = K.new_status(w.trellis.device)
    whole = torch.empty(s * rows * w.N, dtype=torch.float32, device=x.device)
    K.exl3_gemm(x, w, whole, s, status)
    whole = whole.view(s, rows, w.N)
    out = {}
    for r in range(ranks):
        lo, hi = tpfmt.split_width(w.N, r, ranks).cols()
        part_w = K.Exl3Weight(w.trellis[:, lo // 16:hi // 16].contiguous(), w.suh, w.svh[lo:hi].contiguous(), None, w.codebook)
        part = torch.empty(s * rows * (hi - lo), dtype=torch.float32, device=x.device)
        K.exl3_gemm(x, part_w, part, s, status)
        torch.cuda.synchronize()
        K.check_status(status, "shard proof")
        out[r] = bool(torch.equal(part.view(s, rows, hi - lo), whole[:, :, lo:hi]))
    return out


def main(argv=None) -> int:
    import argparse
    import json
    from .. import plan as planmod
    ap = argparse.ArgumentParser(prog="rexl3-shard-proof")
    ap.add_argument("--config", default="dense-27b")
    ap.add_argument("--ranks", type=int, nargs="+", default=[2, 4, 8])
    a = ap.parse_args(argv)
    cfg = planmod.find_config(a.config)
    print(json.dumps({str(R): [p.__dict__ for p in proof_table(dense_shapes(cfg), R)] for R in a.ranks}, indent=1))
    return 0


if __name__ == "__main__":
    import sys
    sys.exit(main())
