"""Causal prefill attention at the 27B geometry (40 query / 8 KV heads of 128, bf16 paged cache): CUDA-event timing of rx_attn_prefill (the
tcgen05 / tensor-memory kernel) and a check of a few rows against a plain fp32 reference.  `--rows N` sets the prompt length (default 8192;
2048 keeps a profiler capture short)."""
import argparse, math, os, sys
import torch
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))))
from rexl3_b200.ops import kernels as K

ap = argparse.ArgumentParser()
ap.add_argument("--rows", type=int, default=8192)
ap.add_argument("--iters", type=int, default=5)
a = ap.parse_args()
hd, n_q, n_kv, T = 128, 40, 8, a.rows
pages = T // 64 + 2
torch.manual_seed(0)
kc = torch.randn(pages, n_kv, 64, hd, device="cuda").to(torch.bfloat16)
vc = torch.randn(pages, n_kv, 64, hd, device="cuda").to(torch.bfloat16)
bt = torch.arange(pages, dtype=torch.int32, device="cuda").view(1, -1).contiguous()
tk, tv = K.KvTensorMap(kc), K.KvTensorMap(vc)
status = K.new_status()
i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")  # noqa: E731
q = torch.randn(T, n_q * hd, device="cuda").to(torch.bfloat16)
out = torch.empty_like(q)
args = (tk, tv, q, bt, i32([0]), i32([0]), i32([T]), i32([0]))
run = lambda: K.attn_prefill(*args, out, 1, T, n_q, n_kv, hd, 1 / math.sqrt(hd), status)  # noqa: E731
for _ in range(2):
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
t = e0.elapsed_time(e1) / a.iters
fl = 4 * T * T * hd * n_q / 2
# plain reference on a few rows
rows = [0, 1, T // 2, T - 1]
kk = kc[:T // 64].permute(1, 0, 2, 3).reshape(n_kv, -1, hd).float()
vv = vc[:T // 64].permute(1, 0, 2, 3).reshape(n_kv, -1, hd).float()
err = 0.0
for r in rows:
    qq = q[r].view(n_q, hd).float()
    for h in range(0, n_q, 7):
        s = (kk[h // (n_q // n_kv), :r + 1] @ qq[h]) / math.sqrt(hd)
        o = torch.softmax(s, 0) @ vv[h // (n_q // n_kv), :r + 1]
        err = max(err, (o - out[r].view(n_q, hd)[h].float()).abs().max().item())
print(f"attn_prefill {T} rows x {n_q} heads: {t:.3f} ms = {fl / t / 1e9:.0f} TFLOP/s (causal FLOPs), max |err| vs fp32 reference {err:.4f}")
