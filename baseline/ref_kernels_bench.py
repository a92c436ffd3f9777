"""Same-box kernel comparator: the reference's own EXL3 linear (its ``mma.sync`` decode kernel, recompiled unchanged
for sm_100 by ``baseline/build_ref_kernels.py``) against this repository's tcgen05 path, on the five matrix shapes of
the 27B-class dense config at 1 / 16 / 64 rows.

Both sides run the whole layer ``y = ((x * suh) H W_q H) * svh``: the reference through ``gb_exl3_linear``
(rot_in -> linear_kernel -> rot_out, crates/cuda/csrc/exl3_linear.cu:691-712, workspace sized by
``gb_exl3_linear_workspace_bytes``), this repository through rx_norm_rot_in (without a norm) -> rx_exl3_gemm ->
rx_finish_store.  Same random trellis (any bit ring is a valid EXL3 tile), same inputs; the two outputs are
compared as a numerics cross-check.  Each side synchronizes right after its first call, before the other side launches
anything, so a device fault is attributed to the side that raised it.  Timing: CUDA events on the launching stream, median of ``--iters`` after
warm-up, weights rotated over several copies so every call streams them from HBM.

    python baseline/ref_kernels_bench.py [--json OUT]
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from rexl3_b200.ops import kernels as K  # noqa: E402

REF_LIB = os.path.join(HERE, "_ref", "libgbkernels.so")
SHAPES = {"qkv": (5120, 7168), "o": (5120, 5120), "gate_up": (5120, 34816), "down": (17408, 5120), "lm_head": (5120, 151936)}
F16, BF16, F32 = 0, 1, 2


def load_ref():
    lib = ctypes.CDLL(REF_LIB)
    v, i, z = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
    lib.gb_exl3_linear_workspace_bytes.restype = z
    lib.gb_exl3_linear_workspace_bytes.argtypes = [i, i, i, i]
    lib.gb_exl3_linear.restype = i
    lib.gb_exl3_linear.argtypes = [v, i, v, v, v, v, v, i, i, i, i, i, i, v, z, v]
    return lib


def median_ms(fn, iters):
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for it in range(iters):
        evs[it][0].record()
        fn(it)
        evs[it][1].record()
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(b) for a, b in evs)
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=12)
    ap.add_argument("--rows", type=int, nargs="*", default=[1, 16, 64])
    ap.add_argument("--shapes", nargs="*", default=list(SHAPES))
    ap.add_argument("--codebook", default="3inst", choices=list(K.CB_ID))
    ap.add_argument("--side", default="both", choices=["both", "own", "ref"],
                    help="which side to run; each side synchronizes after its first call, so a device fault names its side")
    ap.add_argument("--json", default="")
    a = ap.parse_args()
    ref = None
    if a.side != "own":
        if not os.path.exists(REF_LIB):
            sys.exit(f"{REF_LIB} is missing: run python baseline/build_ref_kernels.py --reference DIR first")
        ref = load_ref()
    dev = "cuda"
    torch.manual_seed(0)
    st = torch.cuda.current_stream().cuda_stream
    status = K.new_status()
    out = {}
    sides = ["own", "ref"] if a.side == "both" else [a.side]
    for name in a.shapes:
        k, n = SHAPES[name]
        copies = 2 if name == "lm_head" else 6
        ws = []
        for _ in range(copies):
            tr = torch.randint(-32768, 32767, (k // 16, n // 16, 64), dtype=torch.int16, device=dev)
            suh = (torch.randint(0, 2, (k,), device=dev) * 2 - 1).to(torch.float16)
            svh = (torch.randint(0, 2, (n,), device=dev) * 2 - 1).to(torch.float16)
            ws.append(K.Exl3Weight(tr, suh, svh, None, a.codebook))
        for rows in a.rows:
            x = (torch.randn(rows, k, device=dev) * 0.5).to(torch.bfloat16)
            torch.cuda.synchronize()
            rec = {}
            y = {}
            if "own" in sides:
                splits = K.plan_splits(k, n, True)
                xr = torch.empty(rows, k, dtype=torch.float16, device=dev)
                part = torch.empty(splits * rows * n, dtype=torch.float32, device=dev)
                y_own = torch.empty(rows, n, dtype=torch.float32, device=dev)

                def run_own(it):
                    w = ws[it % copies]
                    K.norm_rot_in(x, None, 0.0, w.suh, xr)
                    K.exl3_gemm(xr, w, part, splits, status)
                    K.finish_store(part, splits, rows, w, y_own)

                run_own(0)
                torch.cuda.synchronize()          # a fault of this side surfaces here, before the other side has launched anything
                K.check_status(status)
                y["own"] = y_own.clone()
                for it in range(3):
                    run_own(it)
                torch.cuda.synchronize()
                rec["own_us"] = median_ms(run_own, a.iters) * 1e3
                K.check_status(status)
            if "ref" in sides:
                ws_bytes = ref.gb_exl3_linear_workspace_bytes(rows, k, n, 4)
                if ws_bytes == 0:
                    raise RuntimeError("the reference refuses this shape")
                wsp = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
                y_ref = torch.empty(rows, n, dtype=torch.float32, device=dev)

                def run_ref(it):
                    w = ws[it % copies]
                    rc = ref.gb_exl3_linear(x.data_ptr(), BF16, w.trellis.data_ptr(), w.suh.data_ptr(), w.svh.data_ptr(), None, y_ref.data_ptr(), F32,
                                            rows, k, n, 4, K.CB_ID[a.codebook], wsp.data_ptr(), ws_bytes, st)
                    if rc != 0:
                        raise RuntimeError(f"gb_exl3_linear returned {rc}")   # stop at the first error: read, do not re-run

                torch.cuda.synchronize()
                run_ref(0)
                torch.cuda.synchronize()          # a fault of the reference's kernels surfaces here and nowhere else
                y["ref"] = y_ref.clone()
                for it in range(3):
                    run_ref(it)
                torch.cuda.synchronize()
                rec["ref_us"] = median_ms(run_ref, a.iters) * 1e3
            gbs = k * n / 2 / 1e3
            line = f"{name:8s} rows {rows:3d}:"
            if "ref_us" in rec:
                rec["ref_GBs"] = gbs / rec["ref_us"]
                line += f"  reference {rec['ref_us']:8.1f} us ({rec['ref_GBs']:6.0f} GB/s)"
            if "own_us" in rec:
                rec["own_GBs"] = gbs / rec["own_us"]
                line += f"  own {rec['own_us']:8.1f} us ({rec['own_GBs']:6.0f} GB/s)"
            if len(y) == 2:
                rec["speedup"] = rec["ref_us"] / rec["own_us"]
                rec["max_abs_diff"] = (y["ref"] - y["own"]).abs().max().item()
                rec["max_abs_ref"] = y["ref"].abs().max().item()
                line += f"  x{rec['speedup']:5.2f}  |diff| {rec['max_abs_diff']:.3e} of {rec['max_abs_ref']:.3e}"
            out[f"{name}_r{rows}"] = rec
            print(line, flush=True)
        del ws
        torch.cuda.empty_cache()
    if a.json:
        json.dump(out, open(a.json, "w"), indent=1)


if __name__ == "__main__":
    main()
