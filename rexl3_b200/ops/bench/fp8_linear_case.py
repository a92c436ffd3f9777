"""FP8 block-scaled linear (E4M3 weights, one E8M0 scale per 32 x 32 tile, bf16 activations) on the tcgen05 kernel: CUDA-event timing at a
prefill size (compute-bound: FLOP/s against the measured cuBLAS bf16 rate) and at decode sizes (weight-streaming: bytes/s against the measured
copy rate), beside torch's bf16 matmul over the dequantised matrix.  Timed calls rotate over three copies of the weights (3 x N x K bytes,
267 MB at the defaults), so every call streams its weights from HBM without an L2 flush in between (a flush by memset leaves the L2 full of
dirty lines whose write-back then competes with the timed kernel).

    python -m rexl3_b200.ops.bench.fp8_linear_case [--n 17408 --k 5120 --rows 1 16 4096]
"""
import argparse, os, sys
import torch
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))))
from rexl3_b200.ops import kernels as K

ap = argparse.ArgumentParser()
ap.add_argument("--n", type=int, default=17408)
ap.add_argument("--k", type=int, default=5120)
ap.add_argument("--rows", type=int, nargs="+", default=[1, 16, 4096])
ap.add_argument("--iters", type=int, default=20)
ap.add_argument("--gemm-peak-tflops", type=float, default=1654.7)
ap.add_argument("--hbm-gbs", type=float, default=6551.0)
a = ap.parse_args()
g = torch.Generator(device="cuda").manual_seed(0)
dense = torch.randn(a.n, a.k, device="cuda", generator=g) * 0.02
w0 = K.Fp8Weight.quantize(dense)
ws = [w0] + [K.Fp8Weight(w0.w.clone(), w0.scales.clone()) for _ in range(2)]
wbs = [w0.dense().to(torch.bfloat16) for _ in range(3)]
st = K.new_status()


def timed(fn):
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    ts = []
    for i in range(a.iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn(i)
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return sorted(ts)[len(ts) // 2] * 1e3


for rows in a.rows:
    x = torch.randn(rows, a.k, device="cuda", generator=g).to(torch.bfloat16)
    out = torch.empty(rows, a.n, dtype=torch.bfloat16, device="cuda")
    t = timed(lambda i: K.fp8_linear(x, ws[i % 3], st, out=out))
    tb = timed(lambda i: torch.matmul(x, wbs[i % 3].T))
    K.check_status(st)
    flops, wbytes = 2.0 * rows * a.k * a.n, a.n * a.k + a.n * a.k // 1024
    print(f"fp8_linear rows {rows} K {a.k} N {a.n}: {t:.1f} us = {flops / t / 1e6:.1f} TFLOP/s ({flops / t / 1e6 / a.gemm_peak_tflops:.3f} of the measured bf16 GEMM rate), "
          f"weights {wbytes / t / 1e3:.0f} GB/s ({wbytes / t / 1e3 / a.hbm_gbs:.3f} of the measured copy rate) | torch bf16 matmul over 2-byte weights {tb:.1f} us")
