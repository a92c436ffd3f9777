"""Sparse attention against dense attention for one latent-attention layer at a long context: `--seqs` sequences of `--ctx` cached tokens, one
decode row each, `--heads` heads.  Dense = rx_mla_attn over the whole context.  Sparse = scores over the pooled index keys + exact top-512
selection + gather of the 2048 (+ tail) selected latent rows into scratch pages + the same attention kernel over those.  CUDA-event timing,
latent cache above L2 by the defaults (4 x 131,072 tokens x 1152 B = 604 MB)."""
import argparse, ctypes, math, os, sys
import torch
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))))
from rexl3_b200.ops import kernels as K
from rexl3_b200.ops import lib as L

ap = argparse.ArgumentParser()
ap.add_argument("--seqs", type=int, default=4)
ap.add_argument("--ctx", type=int, default=131072)
ap.add_argument("--heads", type=int, default=128)
ap.add_argument("--sel-pools", type=int, default=512)
ap.add_argument("--iters", type=int, default=10)
a = ap.parse_args()
lib, st = L.load(), L.stream_ptr
PAGE, D, H, P = 64, 128, 32, 4
blocks = a.ctx // PAGE + 1
pages = a.seqs * blocks
torch.manual_seed(0)
cache = torch.randn(pages, 9, PAGE, 64, device="cuda", dtype=torch.bfloat16)
pool = torch.randn(pages, PAGE // P, D, device="cuda", dtype=torch.bfloat16)
bt = torch.arange(pages, dtype=torch.int32, device="cuda").view(a.seqs, blocks).contiguous()
rows = a.seqs
row_seq = torch.arange(rows, dtype=torch.int32, device="cuda")
pos = torch.full((rows,), a.ctx - 1, dtype=torch.int32, device="cuda")
ctx_len = pos + 1
q = torch.randn(rows, a.heads, 576, device="cuda").to(torch.bfloat16) * 0.2
qi = torch.randn(rows, H * D, device="cuda").to(torch.bfloat16)
wrow = torch.randn(rows, 64, device="cuda").to(torch.bfloat16)
out = torch.empty(rows, a.heads, 512, dtype=torch.bfloat16, device="cuda")
status = K.new_status()
k_stride = a.sel_pools * P + 4
ppr = (k_stride + PAGE - 1) // PAGE
s_stride = (a.ctx // P + 7) // 8 * 8
scores = torch.zeros(rows, s_stride, dtype=torch.float16, device="cuda")
sel = torch.zeros(rows, k_stride, dtype=torch.int32, device="cuda")
flag, sctx = torch.zeros(rows, dtype=torch.int32, device="cuda"), torch.zeros(rows, dtype=torch.int32, device="cuda")
scratch_pages = torch.zeros(rows * ppr, 9, PAGE, 64, dtype=torch.bfloat16, device="cuda")
vbt = torch.arange(rows * ppr, dtype=torch.int32, device="cuda").view(rows, ppr).contiguous()
tc, tsc = K.KvTensorMap(cache), K.KvTensorMap(scratch_pages)
ascr = torch.empty(max(lib.rx_mla_scratch_floats(rows, a.heads, blocks * PAGE), lib.rx_mla_scratch_floats(rows, a.heads, ppr * PAGE)), dtype=torch.float32,
                   device="cuda")
scale = 1.0 / math.sqrt(192)


def dense():
    L.check(lib.rx_mla_attn(tc.ptr, q.data_ptr(), bt.data_ptr(), blocks, row_seq.data_ptr(), ctx_len.data_ptr(), ascr.data_ptr(), rows, a.heads, a.ctx, scale,
                            out.data_ptr(), status.data_ptr(), st()), "dense")


def sparse():
    L.check(lib.rx_dsa_select(qi.data_ptr(), H * D, wrow.data_ptr(), 64, 0, pool.data_ptr(), bt.data_ptr(), blocks, row_seq.data_ptr(), pos.data_ptr(), 2048,
                              1.0 / math.sqrt(H * D), a.sel_pools, a.ctx // P, scores.data_ptr(), s_stride, sel.data_ptr(), k_stride, flag.data_ptr(),
                              sctx.data_ptr(), rows, st()), "select")
    L.check(lib.rx_dsa_gather(cache.data_ptr(), bt.data_ptr(), blocks, row_seq.data_ptr(), sel.data_ptr(), k_stride, flag.data_ptr(), sctx.data_ptr(),
                              scratch_pages.data_ptr(), ppr, rows, st()), "gather")
    L.check(lib.rx_mla_attn_sel(tsc.ptr, q.data_ptr(), vbt.data_ptr(), ppr, row_seq.data_ptr(), sctx.data_ptr(), ascr.data_ptr(), rows, a.heads, ppr * PAGE,
                                scale, out.data_ptr(), status.data_ptr(), flag.data_ptr(), 1, st()), "sparse attn")


def timed(fn):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    K.check_status(status)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    K.check_status(status)
    return e0.elapsed_time(e1) / a.iters * 1e3


td, ts = timed(dense), timed(sparse)
cache_b, pool_b = rows * a.ctx * 1152, rows * (a.ctx // P) * D * 2
print(f"mla attention {rows} rows x ctx {a.ctx} x {a.heads} heads: dense {td:.0f} us ({cache_b / td / 1e3:.0f} GB/s of latent rows), "
      f"sparse (score + select + gather + attend {int(sctx[0])} tokens) {ts:.0f} us (pooled keys {pool_b / 1e6:.1f} MB), ratio {td / ts:.1f}x")
