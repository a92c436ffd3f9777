"""Decode / verify-window attention at the 27B geometry (40 query / 8 KV heads of 128, bf16 paged cache): CUDA-event timing of rx_attn_decode for
`--seqs` sequences of `--ctx` cached tokens with 1 row each (plain decode) and with `--window` adjacent rows each (a speculative verify step
[last, d1 .. dk]).  Rows of one sequence share a CTA's MMA tile, so the window step should cost little more than the one-row step.  The cache
(seqs x ctx x 8 heads x 128 x 2 tensors x 2 bytes) is sized above L2 by the defaults."""
import argparse, math, os, sys
import torch
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))))
from rexl3_b200.ops import kernels as K

ap = argparse.ArgumentParser()
ap.add_argument("--seqs", type=int, default=16)
ap.add_argument("--ctx", type=int, default=4096)
ap.add_argument("--window", type=int, default=5)
ap.add_argument("--iters", type=int, default=20)
a = ap.parse_args()
hd, n_q, n_kv = 128, 40, 8
blocks = (a.ctx + a.window + 63) // 64
pages = a.seqs * blocks
torch.manual_seed(0)
kc = torch.randn(pages, n_kv, 64, hd, device="cuda").to(torch.bfloat16)
vc = torch.randn(pages, n_kv, 64, hd, device="cuda").to(torch.bfloat16)
bt = torch.arange(pages, dtype=torch.int32, device="cuda").view(a.seqs, blocks).contiguous()
tk, tv = K.KvTensorMap(kc), K.KvTensorMap(vc)
status = K.new_status()
suh = torch.ones(n_q * hd, dtype=torch.float16, device="cuda")


def case(w):
    rows = a.seqs * w
    row_seq = torch.arange(a.seqs, dtype=torch.int32, device="cuda").repeat_interleave(w).contiguous()
    ctx = (a.ctx + 1 + torch.arange(w, dtype=torch.int32, device="cuda")).repeat(a.seqs).contiguous()
    q = torch.randn(rows, n_q * hd, device="cuda").to(torch.bfloat16)
    scratch = K.attn_decode_scratch(rows, n_q, hd, blocks * 64)
    out = torch.empty(rows, n_q * hd, dtype=torch.bfloat16, device="cuda")
    xr = torch.empty(rows, n_q * hd, dtype=torch.float16, device="cuda")
    run = lambda: K.attn_decode(tk, tv, q, bt, row_seq, ctx, scratch, n_q, n_kv, hd, blocks * 64, 1 / math.sqrt(hd), suh, xr, out, status,
                                max_seq_rows=w)  # noqa: E731
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    K.check_status(status)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        run()
    e1.record()
    torch.cuda.synchronize()
    K.check_status(status)
    return e0.elapsed_time(e1) / a.iters * 1e3, rows


kv_bytes = a.seqs * a.ctx * n_kv * hd * 2 * 2
t1, r1 = case(1)
tw, rw = case(a.window)
print(f"attn_decode {a.seqs} seqs x ctx {a.ctx}: {r1} rows {t1:.1f} us ({kv_bytes / t1 / 1e3:.0f} GB/s of K/V), {rw} rows {tw:.1f} us "
      f"({kv_bytes / tw / 1e3:.0f} GB/s), ratio {tw / t1:.2f}")
