"""Teacher forward for calibration: run the unquantized dense decoder over calibration token sequences in fp32 and accumulate, for
every linear layer, the second moment of its inputs (the Hessian of that layer's output error).  Counterpart of the reference
quantizer's teacher forward / capture stage (crates/quant/src/lib.rs:1-30, crates/quant/csrc/teacher.cu:1-9), in PyTorch on
whatever device is given.

Keys of the result: (layer, "qkv"), (layer, "o"), (layer, "gate_up"), (layer, "down") and ("lm_head",); each value is a float64
[K, K] matrix over that layer's (padded) inputs, normalised by the number of rows seen.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from ..models.dense import DenseConfig, rope_inv_freq


def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _rope(x, pos, inv_freq):
    ang = pos.to(torch.float32)[:, None] * inv_freq[None, :]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    h = x.shape[-1] // 2
    x1, x2 = x[..., :h], x[..., h:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


class _Moment:
    def __init__(self, k, device):
        self.h = torch.zeros(k, k, dtype=torch.float64, device=device)
        self.rows = 0

    def add(self, x):
        x = x.to(torch.float64)
        self.h += x.T @ x
        self.rows += x.shape[0]

    def result(self):
        return (self.h / max(self.rows, 1)).cpu().numpy()


@torch.no_grad()
def capture_hessians(cfg: DenseConfig, fp: dict, sequences, device="cpu") -> dict:
    """fp: the float weights `quantize_dense` takes.  sequences: iterable of token-id lists (each is one causal context)."""
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(device)  # noqa: E731
    d, F, hd = cfg.d_model, cfg.ffn_padded, cfg.head_dim
    embed = t(fp["embed"])
    layers = [{k: t(v) for k, v in L.items()} for L in fp["layers"]]
    final_norm, inv_freq = t(fp["final_norm"]), torch.from_numpy(rope_inv_freq(cfg)).to(device)
    mom = {}
    for i in range(len(layers)):
        mom[(i, "qkv")], mom[(i, "o")] = _Moment(d, device), _Moment(cfg.n_q * hd, device)
        mom[(i, "gate_up")], mom[(i, "down")] = _Moment(d, device), _Moment(F, device)
    mom[("lm_head",)] = _Moment(d, device)
    g = cfg.n_q // cfg.n_kv
    for seq in sequences:
        ids = torch.as_tensor(list(seq), dtype=torch.long, device=device)
        T = ids.shape[0]
        pos = torch.arange(T, device=device)
        causal = pos[None, :] > pos[:, None]
        h = embed[ids]
        for i, L in enumerate(layers):
            x = _rms(h, L["attn_norm"], cfg.eps)
            mom[(i, "qkv")].add(x)
            q, k, v = (x @ L["q"]).view(T, cfg.n_q, hd), (x @ L["k"]).view(T, cfg.n_kv, hd), (x @ L["v"]).view(T, cfg.n_kv, hd)
            if "q_norm" in L:
                q, k = _rms(q, L["q_norm"], cfg.eps), _rms(k, L["k_norm"], cfg.eps)
            q, k = _rope(q, pos, inv_freq), _rope(k, pos, inv_freq)
            s = torch.einsum("thd,shd->hts", q, k.repeat_interleave(g, dim=1)) / math.sqrt(hd)
            a = torch.einsum("hts,shd->thd", torch.softmax(s.masked_fill(causal[None], float("-inf")), dim=-1), v.repeat_interleave(g, dim=1))
            a = a.reshape(T, -1)
            mom[(i, "o")].add(a)
            h = h + a @ L["o"]
            x = _rms(h, L["ffn_norm"], cfg.eps)
            mom[(i, "gate_up")].add(x)
            act = torch.nn.functional.silu(x @ L["gate"]) * (x @ L["up"])
            if act.shape[1] != F:                       # the stored FFN is padded to a multiple of 128; padded inputs never fire
                act = torch.nn.functional.pad(act, (0, F - act.shape[1]))
            mom[(i, "down")].add(act)
            h = h + act[:, :L["down"].shape[0]] @ L["down"]
        mom[("lm_head",)].add(_rms(h, final_norm, cfg.eps))
    return {k: m.result() for k, m in mom.items()}
