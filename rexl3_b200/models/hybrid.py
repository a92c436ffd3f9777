"""Hybrid decoder family: every layer is a token mixer followed by the dense SwiGLU FFN, and the mixer is one of
  'M'  a Mamba2 (SSD) block,
  'G'  a gated delta net block (delta rule with a scalar decay per head),
  'K'  a Kimi delta attention block (the same rule with a decay per key channel and a sigmoid output gate),
  'A'  GQA attention over the paged KV cache (with or without rotary embedding),
chosen per layer by `HybridConfig.pattern`.  The recurrent kinds keep a constant-size state per sequence.

What it mirrors: the text backbones of the reference's `qwen` family (GQA + GDN, crates/model/src/families/qwen.rs, kernels
crates/cuda/csrc/gdn.cu:1-25), its KDA layers (crates/cuda/csrc/kda.cu) and its `nemotron_h_omni` family (Mamba2 + NoPE GQA,
crates/model/src/families/nemotron_h_omni/mod.rs:58-251, oracle ssm_ref.rs, kernels crates/cuda/csrc/nemotron_ssm.cu:1-45), with
this engine's own executor: a recurrent layer is in_proj (EXL3 GEMM) -> finish to f32 rows -> conv + recurrence + gated norm
(`ops/csrc/ssm.cu`) -> rotation -> out_proj (EXL3 GEMM), whose partials feed the same fused add + norm + rotate finish as an
attention layer's o_proj.

Recurrent state lives in two pools per recurrent layer, indexed by the engine's sequence slot.  A row at position 0 restarts the
state, so slots are reused without a reset call.  On the GPU every row fed is committed: the CUDA backend over this executor offers
no drafts and no prefix cache.  The fp32 oracle (`ReferenceHybrid`, behind `engine.cpu_backend.CpuHybridBackend`) can snapshot and
restore a sequence, which is how drafts, prompt scoring and the prefix cache work over recurrent layers there.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

from ..format import exl3
from .dense import (DenseConfig, DenseGPU, HostLinear, HostWeights, ReferenceDense, _bf16_round, random_linear, rope_inv_freq)


@dataclass
class HybridConfig(DenseConfig):
    pattern: str = ""            # one letter per layer: 'M' Mamba2, 'G' gated delta net, 'K' Kimi delta attention, 'A' attention
    ssm_heads: int = 0
    ssm_head_dim: int = 64
    ssm_groups: int = 1
    ssm_state: int = 128
    conv_k: int = 4
    nope: bool = True            # attention layers without rotary embedding
    gdn_k_heads: int = 0         # gated delta net: key heads x 128 (value head h reads key head h // (v_heads / k_heads))
    gdn_v_heads: int = 0         # value heads x 128

    @property
    def d_inner(self) -> int:
        return self.ssm_heads * self.ssm_head_dim

    @property
    def conv_channels(self) -> int:
        return self.d_inner + 2 * self.ssm_groups * self.ssm_state

    @property
    def in_proj_width(self) -> int:
        """z | x | B | C | dt, padded up to a multiple of 128 columns (the padding columns are exactly zero)."""
        return (2 * self.d_inner + 2 * self.ssm_groups * self.ssm_state + self.ssm_heads + 127) // 128 * 128

    @property
    def gdn_inner(self) -> int:
        return self.gdn_v_heads * 128

    @property
    def gdn_conv_channels(self) -> int:
        return (2 * self.gdn_k_heads + self.gdn_v_heads) * 128

    @property
    def gdn_proj_width(self) -> int:
        """z | q | k | v | b | a, padded up to a multiple of 128 columns."""
        return (self.gdn_inner + self.gdn_conv_channels + 2 * self.gdn_v_heads + 127) // 128 * 128

    @property
    def kda_proj_width(self) -> int:
        """z | q | k | v | b | a (one decay input per key channel), padded up to a multiple of 128 columns."""
        return (self.gdn_inner + self.gdn_conv_channels + self.gdn_v_heads + self.gdn_inner + 127) // 128 * 128

    def delta_proj_width(self, kind: str) -> int:
        return self.kda_proj_width if kind == "K" else self.gdn_proj_width

    def gdn_layers(self):
        """Layers with a delta-rule mixer ('G' or 'K'): they share head geometry, pools and kernels."""
        return [i for i, c in enumerate(self.pattern) if c in "GK"]

    def mamba_layers(self):
        return [i for i, c in enumerate(self.pattern) if c == "M"]

    def attn_layers(self):
        return [i for i, c in enumerate(self.pattern) if c == "A"]

    def validate(self) -> None:
        if len(self.pattern) != self.n_layers or set(self.pattern) - {"M", "A", "G", "K"}:
            raise ValueError("pattern needs one of 'M' / 'G' / 'K' / 'A' per layer")
        if self.conv_k != 4:
            raise ValueError("the conv kernel is built for width 4")
        if "M" in self.pattern:
            if self.ssm_head_dim != 64 or self.ssm_state != 128:
                raise ValueError("the Mamba2 kernels are built for head_dim 64, state 128")
            if self.ssm_heads <= 0 or self.ssm_heads % self.ssm_groups or self.d_inner % 128:
                raise ValueError("ssm_heads must be a multiple of ssm_groups and even")
        if ("G" in self.pattern or "K" in self.pattern) and (self.gdn_k_heads <= 0 or self.gdn_v_heads % self.gdn_k_heads):
            raise ValueError("gdn_v_heads must be a positive multiple of gdn_k_heads")

    def weight_params(self) -> int:
        ffn = 3 * self.d_model * self.ffn_padded
        attn = self.d_model * self.qkv_width + self.n_q * self.head_dim * self.d_model
        ssm = self.d_model * self.in_proj_width + self.d_inner * self.d_model
        delta = sum(self.d_model * self.delta_proj_width(self.pattern[i]) + self.gdn_inner * self.d_model + ffn for i in self.gdn_layers())
        return len(self.attn_layers()) * (attn + ffn) + len(self.mamba_layers()) * (ssm + ffn) + delta + self.vocab_padded * self.d_model

    def state_bytes_per_slot(self) -> int:
        return (len(self.mamba_layers()) * 4 * (self.ssm_heads * self.ssm_head_dim * self.ssm_state + 3 * self.conv_channels)
                + len(self.gdn_layers()) * 4 * (self.gdn_v_heads * 128 * 128 + 3 * self.gdn_conv_channels))

    def kv_bytes_per_token(self, elem_bytes: int = 2) -> int:
        return 2 * self.n_kv * self.head_dim * elem_bytes * len(self.attn_layers())


CONFIGS = {
    # the reference family's block geometry (128 heads x 64, state 128, 8 groups; GQA 32q / 2kv x 128) as a dense-FFN hybrid
    "hybrid-h-56l": HybridConfig(n_layers=56, d_model=4096, n_q=32, n_kv=2, head_dim=128, ffn=14336, vocab=131072, bits=4.0, name="hybrid-h-56l",
                                 pattern="MMMMMMA" * 8, ssm_heads=128, ssm_groups=8),
    # the reference's flagship layout (three gated-delta-net layers, then one attention layer, x16; 16 key / 48 value heads x 128) on
    # the 27B-class dense geometry
    "gdn-hybrid-27b": HybridConfig(n_layers=64, d_model=5120, n_q=40, n_kv=8, head_dim=128, ffn=17408, vocab=151936, rope_theta=1e6, bits=4.0,
                                   name="gdn-hybrid-27b", pattern="GGGA" * 16, nope=False, gdn_k_heads=16, gdn_v_heads=48),
    "test-hybrid-gdn": HybridConfig(n_layers=4, d_model=512, n_q=8, n_kv=2, head_dim=128, ffn=1024, vocab=4096, bits=4.0, name="test-hybrid-gdn",
                                    pattern="GAMG", nope=False, ssm_heads=16, ssm_groups=2, gdn_k_heads=2, gdn_v_heads=4),
    "test-hybrid-kda": HybridConfig(n_layers=3, d_model=512, n_q=8, n_kv=2, head_dim=128, ffn=1024, vocab=4096, bits=4.0, name="test-hybrid-kda",
                                    pattern="KAK", nope=True, gdn_k_heads=4, gdn_v_heads=4),
    # CPU plumbing model of the family (one layer of each recurrent kind and one attention layer; quantizes in seconds on the host)
    "tiny-hybrid": HybridConfig(n_layers=3, d_model=128, n_q=2, n_kv=1, head_dim=64, ffn=128, vocab=512, bits=4.0, name="tiny-hybrid", pattern="MGA",
                                ssm_heads=2, ssm_groups=1, gdn_k_heads=1, gdn_v_heads=1),
    "test-hybrid": HybridConfig(n_layers=4, d_model=512, n_q=8, n_kv=2, head_dim=128, ffn=1024, vocab=4096, bits=4.0, name="test-hybrid",
                                pattern="MAMM", ssm_heads=16, ssm_groups=2),
}


@dataclass
class HostMambaLayer:
    attn_norm: np.ndarray
    in_proj: HostLinear
    out_proj: HostLinear
    conv_w: np.ndarray           # [C, 4], tap 3 multiplies the current row
    conv_b: np.ndarray           # [C]
    dt_bias: np.ndarray          # [H]
    a_log: np.ndarray            # [H]; A = -exp(a_log)
    d_skip: np.ndarray           # [H]
    norm_w: np.ndarray           # [d_inner]
    ffn_norm: np.ndarray
    gate_up: HostLinear
    down: HostLinear


@dataclass
class HostGdnLayer:
    attn_norm: np.ndarray
    in_proj: HostLinear          # z | q | k | v | b | a
    out_proj: HostLinear
    conv_w: np.ndarray           # [C, 4]
    conv_b: np.ndarray           # [C]
    dt_bias: np.ndarray          # [Hv]; Kimi delta attention: [Hv * 128], one per key channel
    a_log: np.ndarray            # [Hv]; A = -exp(a_log)
    norm_w: np.ndarray           # [128], shared by the heads
    ffn_norm: np.ndarray
    gate_up: HostLinear
    down: HostLinear
    kda: bool = False            # per-key-channel decay and a sigmoid output gate


def random_weights(cfg: HybridConfig, seed: int = 0) -> HostWeights:
    """Random-init hybrid weights (valid random EXL3 tensors; SSM parameters in their usual ranges)."""
    from .dense import HostLayer
    cfg.validate()
    rng = np.random.default_rng(seed)
    d, F, DI, H, C = cfg.d_model, cfg.ffn_padded, cfg.d_inner, cfg.ssm_heads, cfg.conv_channels
    s_in = 1.0 / math.sqrt(d)
    w = HostWeights(cfg, _bf16_round(rng.normal(0, 1.0, size=(cfg.vocab, d)).astype(np.float32)))
    nrm = lambda n: _bf16_round(1.0 + 0.1 * rng.normal(size=n))  # noqa: E731
    for kind in cfg.pattern:
        gu = random_linear(d, 2 * F, cfg.bits, rng, cfg.codebook, s_in)
        if F != cfg.ffn:
            gu.svh[cfg.ffn:F] = 0
            gu.svh[F + cfg.ffn:] = 0
        down = random_linear(F, d, cfg.bits, rng, cfg.codebook, 0.5 / math.sqrt(F), zero_rows_from=cfg.ffn if F != cfg.ffn else None)
        if kind == "A":
            qkv = random_linear(d, cfg.qkv_width, cfg.bits, rng, cfg.codebook, s_in)
            o = random_linear(cfg.n_q * cfg.head_dim, d, cfg.bits, rng, cfg.codebook, 0.5 / math.sqrt(cfg.n_q * cfg.head_dim))
            w.layers.append(HostLayer(nrm(d), qkv, o, nrm(d), gu, down))
            continue
        if kind in "GK":
            GI, GC, Hv, kda = cfg.gdn_inner, cfg.gdn_conv_channels, cfg.gdn_v_heads, kind == "K"
            real, wp = GI + GC + Hv + (GI if kda else Hv), cfg.delta_proj_width(kind)
            ip = random_linear(d, wp, cfg.bits, rng, cfg.codebook, s_in, zero_cols_from=real if real != wp else None)
            op = random_linear(GI, d, cfg.bits, rng, cfg.codebook, 0.5 / math.sqrt(GI))
            w.layers.append(HostGdnLayer(
                nrm(d), ip, op, _bf16_round(rng.normal(0, 0.5, size=(GC, 4))), _bf16_round(rng.normal(0, 0.1, size=GC)),
                rng.uniform(-2.0, 0.0, size=GI if kda else Hv).astype(np.float32), np.log(rng.uniform(0.5, 4.0, size=Hv)).astype(np.float32), nrm(128),
                nrm(d), gu, down, kda))
            continue
        real = 2 * DI + 2 * cfg.ssm_groups * cfg.ssm_state + H
        ip = random_linear(d, cfg.in_proj_width, cfg.bits, rng, cfg.codebook, s_in, zero_cols_from=real if real != cfg.in_proj_width else None)
        op = random_linear(DI, d, cfg.bits, rng, cfg.codebook, 0.5 / math.sqrt(DI))
        w.layers.append(HostMambaLayer(
            nrm(d), ip, op, _bf16_round(rng.normal(0, 0.5, size=(C, 4))), _bf16_round(rng.normal(0, 0.1, size=C)),
            rng.uniform(-3.0, -1.0, size=H).astype(np.float32), np.log(rng.uniform(1.0, 16.0, size=H)).astype(np.float32),
            rng.normal(1.0, 0.1, size=H).astype(np.float32), nrm(DI), nrm(d), gu, down))
    w.final_norm = nrm(d)
    w.lm_head = random_linear(d, cfg.vocab_padded, cfg.head_bits or cfg.bits, rng, cfg.codebook, s_in,
                              zero_cols_from=cfg.vocab if cfg.vocab_padded != cfg.vocab else None)
    return w


# ====================================================================================================== reference
class ReferenceHybrid(ReferenceDense):
    """fp32 oracle: the dense reference with a per-layer mixer switch and a token-by-token Mamba2 recurrence."""

    def __init__(self, w: HostWeights, device="cpu", dtype=torch.float32):
        self.cfg = cfg = w.cfg
        self.device, self.dtype = device, dtype
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(device=device, dtype=dtype)  # noqa: E731
        self.embed = t(w.embed)
        self.layers = []
        for lay in w.layers:
            L = dict(attn_norm=t(lay.attn_norm), ffn_norm=t(lay.ffn_norm), gate_up=t(lay.gate_up.dense()), down=t(lay.down.dense()), q_norm=None, k_norm=None)
            if isinstance(lay, HostMambaLayer):
                L.update(kind="M", in_proj=t(lay.in_proj.dense()), o=t(lay.out_proj.dense()), conv_w=t(lay.conv_w), conv_b=t(lay.conv_b),
                         dt_bias=t(lay.dt_bias), a_neg=-torch.exp(t(lay.a_log)), d_skip=t(lay.d_skip), norm_w=t(lay.norm_w))
            elif isinstance(lay, HostGdnLayer):
                L.update(kind="K" if lay.kda else "G", in_proj=t(lay.in_proj.dense()), o=t(lay.out_proj.dense()), conv_w=t(lay.conv_w), conv_b=t(lay.conv_b),
                         dt_bias=t(lay.dt_bias), a_neg=-torch.exp(t(lay.a_log)), norm_w=t(lay.norm_w))
            else:
                L.update(kind="A", qkv=t(lay.qkv.dense()), o=t(lay.o.dense()))
            self.layers.append(L)
        self.final_norm = t(w.final_norm)
        self.lm_head = t(w.lm_head.dense())[:, :cfg.vocab]
        self.inv_freq = torch.from_numpy(rope_inv_freq(cfg)).to(device)
        if cfg.nope:
            self.inv_freq.zero_()
        self.kv = {}
        self.ssm = {}          # (seq, layer) -> (conv history [3, C], state [H, P, N])
        self.seq_len = {}

    def reset(self, seq=None):
        super().reset(seq)
        for k in [k for k in self.ssm if seq is None or k[0] == seq]:
            del self.ssm[k]
        if seq is None:
            self.seq_len.clear()
        else:
            self.seq_len.pop(seq, None)

    @torch.no_grad()
    def forward_seq(self, seq, tokens, start: int, n_layers: int | None = None):
        out = super().forward_seq(seq, tokens, start, n_layers)
        self.seq_len[seq] = start + len(tokens)
        return out

    def truncate(self, seq, length: int):
        """Only the no-op is possible: a recurrent state cannot be rolled back (callers that must undo rows use snapshot / restore)."""
        if length != self.seq_len.get(seq, 0):
            raise NotImplementedError("a recurrent state cannot be rolled back")

    def snapshot(self, seq):
        """Everything `seq` has accumulated (attention KV, conv histories, recurrent states, length), for `restore`."""
        return (self.seq_len.get(seq, 0), None if seq not in self.kv else [(k.clone(), v.clone()) for k, v in self.kv[seq]],
                {k: (c.clone(), s.clone()) for k, (c, s) in self.ssm.items() if k[0] == seq})

    def restore(self, seq, snap) -> None:
        n, kv, ssm = snap
        self.reset(seq)
        self.seq_len[seq] = n
        if kv is not None:
            self.kv[seq] = [(k.clone(), v.clone()) for k, v in kv]
        for k, (c, s) in ssm.items():
            self.ssm[k] = (c.clone(), s.clone())

    def _mix(self, li, L, h, pos, seq, start):
        if L["kind"] == "A":
            return super()._mix(li, L, h, pos, seq, start)
        if L["kind"] in "GK":
            return self._gdn(li, L, h, seq, start, L["kind"] == "K")
        cfg = self.cfg
        T, H, P, G, N, DI, C = h.shape[0], cfg.ssm_heads, cfg.ssm_head_dim, cfg.ssm_groups, cfg.ssm_state, cfg.d_inner, cfg.conv_channels
        proj = self._rms(h, L["attn_norm"], cfg.eps) @ L["in_proj"]
        z, xbc, dt = proj[:, :DI], proj[:, DI:DI + C], proj[:, DI + C:DI + C + H]
        if start == 0 or (seq, li) not in self.ssm:
            hist, S = torch.zeros(3, C, device=h.device, dtype=h.dtype), torch.zeros(H, P, N, device=h.device, dtype=h.dtype)
        else:
            hist, S = self.ssm[(seq, li)]
        full = torch.cat([hist, xbc])
        conv = L["conv_b"][None, :] + sum(L["conv_w"][:, j][None, :] * full[j:j + T] for j in range(4))
        act = torch.nn.functional.silu(conv)
        xs = act[:, :DI].view(T, H, P)
        Bm = act[:, DI:DI + G * N].view(T, G, N).repeat_interleave(H // G, dim=1)
        Cm = act[:, DI + G * N:].view(T, G, N).repeat_interleave(H // G, dim=1)
        dt = torch.nn.functional.softplus(dt + L["dt_bias"][None, :])
        dA = torch.exp(dt * L["a_neg"][None, :])
        y = torch.empty(T, H, P, device=h.device, dtype=h.dtype)
        for t_ in range(T):
            S = S * dA[t_][:, None, None] + (xs[t_] * dt[t_][:, None])[:, :, None] * Bm[t_][:, None, :]
            y[t_] = (S * Cm[t_][:, None, :]).sum(-1) + L["d_skip"][:, None] * xs[t_]
        self.ssm[(seq, li)] = (full[-3:].clone(), S)
        g = (y.reshape(T, DI) * torch.nn.functional.silu(z)).view(T, G, DI // G)
        g = g * torch.rsqrt(g.pow(2).mean(-1, keepdim=True) + cfg.eps)
        return (g.reshape(T, DI) * L["norm_w"]) @ L["o"]


    def _gdn(self, li, L, h, seq, start, kda=False):
        """Gated delta net, token by token (the public recurrent form: decay, delta-rule write, read, per-head gated RMSNorm).  `kda`: the decay
        is a vector over the key channels and the output gate a sigmoid (Kimi delta attention)."""
        cfg, F = self.cfg, torch.nn.functional
        T, Hk, Hv, D, DI, C = h.shape[0], cfg.gdn_k_heads, cfg.gdn_v_heads, 128, cfg.gdn_inner, cfg.gdn_conv_channels
        proj = self._rms(h, L["attn_norm"], cfg.eps) @ L["in_proj"]
        z, qkv, b, a = proj[:, :DI], proj[:, DI:DI + C], proj[:, DI + C:DI + C + Hv], proj[:, DI + C + Hv:DI + C + Hv + (DI if kda else Hv)]
        if start == 0 or (seq, li) not in self.ssm:
            hist, S = torch.zeros(3, C, device=h.device, dtype=h.dtype), torch.zeros(Hv, D, D, device=h.device, dtype=h.dtype)
        else:
            hist, S = self.ssm[(seq, li)]
        full = torch.cat([hist, qkv])
        act = F.silu(L["conv_b"][None, :] + sum(L["conv_w"][:, j][None, :] * full[j:j + T] for j in range(4)))
        l2 = lambda x: x * torch.rsqrt(x.pow(2).sum(-1, keepdim=True) + 1e-6)  # noqa: E731
        q = (l2(act[:, :Hk * D].view(T, Hk, D)) / math.sqrt(D)).repeat_interleave(Hv // Hk, dim=1)
        k = l2(act[:, Hk * D:2 * Hk * D].view(T, Hk, D)).repeat_interleave(Hv // Hk, dim=1)
        v = act[:, 2 * Hk * D:].view(T, Hv, D)
        if kda:        # [T, Hv, 1, D]: one factor per key channel i
            decay = torch.exp(L["a_neg"][None, :, None] * F.softplus(a + L["dt_bias"][None, :]).view(T, Hv, D))[:, :, None, :]
        else:
            decay = torch.exp(L["a_neg"][None, :] * F.softplus(a + L["dt_bias"][None, :]))[:, :, None, None]
        beta = torch.sigmoid(b)
        o = torch.empty(T, Hv, D, device=h.device, dtype=h.dtype)
        for t_ in range(T):                                   # S[h, j (value), i (key)]
            S = S * decay[t_]
            kv = (S * k[t_][:, None, :]).sum(-1)
            S = S + ((v[t_] - kv) * beta[t_][:, None])[:, :, None] * k[t_][:, None, :]
            o[t_] = (S * q[t_][:, None, :]).sum(-1)
        self.ssm[(seq, li)] = (full[-3:].clone(), S)
        o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + cfg.eps) * L["norm_w"][None, None, :]
        return (o.reshape(T, DI) * (torch.sigmoid(z) if kda else F.silu(z))) @ L["o"]


def delta_state_canonical(pool: torch.Tensor) -> torch.Tensor:
    """A delta-net state pool [slots, Hv, 128, 128] as stored (the kernel's access order: [warp = j / 16][step s][lane = 2 (j % 16) + half][e],
    holding S[value j][key i] with i = 64 half + 4 s + e) -> canonical [slots, Hv, value j, key i]."""
    S, Hv = pool.shape[0], pool.shape[1]
    return pool.reshape(S, Hv, 8, 16, 16, 2, 4).permute(0, 1, 2, 4, 5, 3, 6).reshape(S, Hv, 128, 128)


# ====================================================================================================== sm_100a executor
class HybridGPU(DenseGPU):
    """One B200.  Attention layers run the dense executor's mixer; Mamba2, gated-delta-net and Kimi-delta-attention layers run the recurrent
    branch of `_mixer` (in_proj GEMM -> f32 rows -> conv + recurrence + gated norm kernels -> rotation -> out_proj GEMM).  A recurrent layer's
    in_proj / out_proj sit under the keys "qkv" / "o" of its layer dict as well, so the shared layer loop finds each layer's input rotation
    and output scales.  State pools (`conv_pool`, `ssm_pool`) are indexed by the engine's sequence slot; `state_view` gives them in canonical
    order."""

    def __init__(self, w: "HostWeights | HybridConfig", num_pages: int, max_rows: int = 256, max_seqs: int = 64, max_blocks_per_seq: int = 256,
                 device="cuda", max_prefill_rows: int = 8192, seed: int = 0, kv_dtype: str = "bf16"):
        cfg = w if isinstance(w, HybridConfig) else w.cfg
        cfg.validate()
        super().__init__(w, num_pages, max_rows, max_seqs, max_blocks_per_seq, device, max_prefill_rows, seed, kv_dtype)
        if cfg.nope:
            self.inv_freq.zero_()
        H, P, N, C = cfg.ssm_heads, cfg.ssm_head_dim, cfg.ssm_state, cfg.conv_channels
        self.conv_pool = {li: torch.zeros(max_seqs, 3, C, dtype=torch.float32, device=device) for li in cfg.mamba_layers()}
        self.ssm_pool = {li: torch.zeros(max_seqs, H, P, N, dtype=torch.float32, device=device) for li in cfg.mamba_layers()}
        for li in cfg.gdn_layers():
            self.conv_pool[li] = torch.zeros(max_seqs, 3, cfg.gdn_conv_channels, dtype=torch.float32, device=device)
            self.ssm_pool[li] = torch.zeros(max_seqs, cfg.gdn_v_heads, 128, 128, dtype=torch.float32, device=device)
        self.ssm_mode = self.K.SCAN_FINAL       # how the recurrent layers treat the rows of the next forward (see `enable_record`)
        self.rec_proj, self.rec_xbc, self.rec_rows = {}, {}, 0

    # ------------------------------------------------------------------ record / commit split of the recurrent layers
    def enable_record(self, rows: int) -> None:
        """Buffers that let a window of up to `rows` rows be fed without touching the pools (`ssm_mode = SCAN_RECORD`): every recurrent layer
        keeps that window's in_proj rows and post-conv rows, and `commit_rows` later replays the accepted prefix of each sequence from them
        (the reference's record / commit split, crates/cuda/csrc/gdn.cu:253-322).  Costs (proj width + conv channels) * 4 bytes per row
        and layer."""
        cfg, dev = self.cfg, self.device
        if rows <= self.rec_rows:
            return
        for li, L in enumerate(self.layers):
            if L["kind"] == "A":
                continue
            wp = cfg.in_proj_width if L["kind"] == "M" else cfg.delta_proj_width(L["kind"])
            wc = cfg.conv_channels if L["kind"] == "M" else cfg.gdn_conv_channels
            self.rec_proj[li] = torch.empty(rows, wp, dtype=torch.float32, device=dev)
            self.rec_xbc[li] = torch.empty(rows * wc, dtype=torch.float32, device=dev)
        self.rec_rows = rows

    def record_bytes(self) -> int:
        return sum(t.numel() * 4 for t in self.rec_proj.values()) + sum(t.numel() * 4 for t in self.rec_xbc.values())

    def commit_rows(self, M: int, row_seq, positions, seg_start, seg_len, nseg: int) -> None:
        """Advance the pools over the first seg_len[i] rows of segment i of the last recorded window (rows, row_seq and positions as they were
        fed).  One launch per recurrent layer; the arithmetic is the window's own, so the pools end up as a serial decode leaves them."""
        cfg, K = self.cfg, self.K
        for li, L in enumerate(self.layers):
            if L["kind"] == "A":
                continue
            proj = self.rec_proj[li][:M]
            if L["kind"] in "GK":
                K.gdn_mixer(proj, M, cfg.gdn_k_heads, cfg.gdn_v_heads, 128, row_seq, positions, seg_start, seg_len, nseg, L["conv_w"], L["conv_b"],
                            L["dt_bias"], L["a_neg"], L["norm_w"], cfg.eps, self.conv_pool[li], self.ssm_pool[li], self.rec_xbc[li], self.ssm_out,
                            kda=L["kind"] == "K", mode=K.SCAN_COMMIT, y32=self.ssm_y)
            else:
                K.ssm_mixer(proj, M, cfg.ssm_heads, cfg.ssm_head_dim, cfg.ssm_groups, cfg.ssm_state, row_seq, positions, seg_start, seg_len, nseg,
                            L["conv_w"], L["conv_b"], L["dt_bias"], L["a_neg"], L["d_skip"], L["norm_w"], cfg.eps, self.conv_pool[li],
                            self.ssm_pool[li], self.rec_xbc[li], self.ssm_y, self.ssm_out, mode=K.SCAN_COMMIT)

    def _kv_layers(self):
        return self.cfg.attn_layers()

    def _gemm_shapes(self) -> dict:
        cfg = self.cfg
        s = super()._gemm_shapes()
        if "M" in cfg.pattern:
            s.update(in_proj=(cfg.d_model, cfg.in_proj_width), out_proj=(cfg.d_inner, cfg.d_model))
        if "G" in cfg.pattern:
            s.update(gdn_in=(cfg.d_model, cfg.gdn_proj_width), gdn_out=(cfg.gdn_inner, cfg.d_model))
        if "K" in cfg.pattern:
            s.update(kda_in=(cfg.d_model, cfg.kda_proj_width), gdn_out=(cfg.gdn_inner, cfg.d_model))
        return s

    def _alloc_scratch(self, R: int):
        super()._alloc_scratch(R)
        cfg, dev = self.cfg, self.device
        m, g = "M" in cfg.pattern, bool(cfg.gdn_layers())
        wp = max(cfg.in_proj_width if m else 0, cfg.gdn_proj_width if "G" in cfg.pattern else 0, cfg.kda_proj_width if "K" in cfg.pattern else 0)
        wc = max(cfg.conv_channels if m else 0, cfg.gdn_conv_channels if g else 0)
        wi = max(cfg.d_inner if m else 0, cfg.gdn_inner if g else 0)
        self.ssm_proj = torch.empty(R * wp, dtype=torch.float32, device=dev)       # flat: each layer kind views its own row width
        self.ssm_xbc = torch.empty(R * wc, dtype=torch.float32, device=dev)
        self.ssm_y = torch.empty(R * max(cfg.d_inner if m else 1, cfg.gdn_inner if g else 1), dtype=torch.float32, device=dev)
        self.ssm_out = torch.empty(R * wi, dtype=torch.bfloat16, device=dev)

    # ------------------------------------------------------------------ weights
    def _mamba_dict(self, attn_norm, ip, op, conv_w, conv_b, dt_bias, a_neg, d_skip, norm_w, ffn_norm, gu, dn):
        return dict(kind="M", attn_norm=attn_norm, qkv=ip, o=op, in_proj=ip, out_proj=op, conv_w=conv_w, conv_b=conv_b, dt_bias=dt_bias, a_neg=a_neg,
                    d_skip=d_skip, norm_w=norm_w, ffn_norm=ffn_norm, gate_up=gu, down=dn, q_norm=None, k_norm=None)

    def _upload_host(self, w: HostWeights) -> None:
        K, device = self.K, self.device
        dev = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(device=device, dtype=dt)  # noqa: E731
        up = lambda l: K.Exl3Weight.from_numpy(l.trellis, l.suh, l.svh, l.bias, l.codebook, device)  # noqa: E731
        bf, f32 = torch.bfloat16, torch.float32
        self.embed = dev(w.embed, bf)
        self.layers = []
        for lay in w.layers:
            if isinstance(lay, HostGdnLayer):
                ip, op = up(lay.in_proj), up(lay.out_proj)
                self.layers.append(dict(kind="K" if lay.kda else "G", attn_norm=dev(lay.attn_norm, bf), qkv=ip, o=op, in_proj=ip, out_proj=op, conv_w=dev(lay.conv_w, bf),
                                        conv_b=dev(lay.conv_b, bf), dt_bias=dev(lay.dt_bias, f32), a_neg=-torch.exp(dev(lay.a_log, f32)),
                                        norm_w=dev(lay.norm_w, bf), ffn_norm=dev(lay.ffn_norm, bf), gate_up=up(lay.gate_up), down=up(lay.down),
                                        q_norm=None, k_norm=None))
            elif isinstance(lay, HostMambaLayer):
                self.layers.append(self._mamba_dict(dev(lay.attn_norm, bf), up(lay.in_proj), up(lay.out_proj), dev(lay.conv_w, bf), dev(lay.conv_b, bf),
                                                    dev(lay.dt_bias, f32), -torch.exp(dev(lay.a_log, f32)), dev(lay.d_skip, f32), dev(lay.norm_w, bf),
                                                    dev(lay.ffn_norm, bf), up(lay.gate_up), up(lay.down)))
            else:
                self.layers.append(dict(kind="A", attn_norm=dev(lay.attn_norm, bf), qkv=up(lay.qkv), o=up(lay.o), ffn_norm=dev(lay.ffn_norm, bf),
                                        gate_up=up(lay.gate_up), down=up(lay.down), q_norm=None, k_norm=None))
        self.final_norm = dev(w.final_norm, bf)
        self.lm_head = up(w.lm_head)

    def _load_random(self, seed: int) -> None:
        cfg, K, device = self.cfg, self.K, self.device
        g = torch.Generator(device=device).manual_seed(seed)
        tw = exl3.Bits.of(cfg.bits).tile_words
        cb = cfg.codebook if exl3.Bits.of(cfg.bits).is_integer else "mul1"

        def lin(k, n, scale, words=tw, real_n=None):
            tr = torch.randint(-32768, 32768, (k // 16, n // 16, words), dtype=torch.int16, device=device, generator=g)
            sg = lambda m: (torch.randint(0, 2, (m,), device=device, generator=g) * 2 - 1)  # noqa: E731
            wt = K.Exl3Weight(tr, sg(k).to(torch.float16), (sg(n) * scale).to(torch.float16), None, cb)
            if real_n is not None and real_n != n:
                wt.svh[real_n:] = 0
            return wt

        rn = lambda *s: torch.randn(*s, device=device, generator=g)  # noqa: E731
        ru = lambda n, lo, hi: lo + (hi - lo) * torch.rand(n, device=device, generator=g)  # noqa: E731
        norm = lambda n=cfg.d_model: (1.0 + 0.1 * rn(n)).to(torch.bfloat16)  # noqa: E731
        d, F, HQ, DI, H, C = cfg.d_model, cfg.ffn_padded, cfg.n_q * cfg.head_dim, cfg.d_inner, cfg.ssm_heads, cfg.conv_channels
        self.embed = rn(cfg.vocab, d).to(torch.bfloat16)
        self.layers = []
        for kind in cfg.pattern:
            gu = lin(d, 2 * F, 1.0 / math.sqrt(d))
            dn = lin(F, d, 0.5 / math.sqrt(F))
            if F != cfg.ffn:
                gu.svh[cfg.ffn:F] = 0
                gu.svh[F + cfg.ffn:] = 0
                dn.suh[cfg.ffn:] = 0
            if kind == "A":
                self.layers.append(dict(kind="A", attn_norm=norm(), qkv=lin(d, cfg.qkv_width, 1.0 / math.sqrt(d)), o=lin(HQ, d, 0.5 / math.sqrt(HQ)),
                                        ffn_norm=norm(), gate_up=gu, down=dn, q_norm=None, k_norm=None))
                continue
            if kind in "GK":
                GI, GC, Hv, kda = cfg.gdn_inner, cfg.gdn_conv_channels, cfg.gdn_v_heads, kind == "K"
                ip = lin(d, cfg.delta_proj_width(kind), 1.0 / math.sqrt(d), real_n=GI + GC + Hv + (GI if kda else Hv))
                op = lin(GI, d, 0.5 / math.sqrt(GI))
                self.layers.append(dict(kind=kind, attn_norm=norm(), qkv=ip, o=op, in_proj=ip, out_proj=op, conv_w=(0.5 * rn(GC, 4)).to(torch.bfloat16),
                                        conv_b=(0.1 * rn(GC)).to(torch.bfloat16), dt_bias=ru(GI if kda else Hv, -2.0, 0.0), a_neg=-ru(Hv, 0.5, 4.0),
                                        norm_w=norm(128),
                                        ffn_norm=norm(), gate_up=gu, down=dn, q_norm=None, k_norm=None))
                continue
            ip = lin(d, cfg.in_proj_width, 1.0 / math.sqrt(d), real_n=2 * DI + 2 * cfg.ssm_groups * cfg.ssm_state + H)
            op = lin(DI, d, 0.5 / math.sqrt(DI))
            self.layers.append(self._mamba_dict(norm(), ip, op, (0.5 * rn(C, 4)).to(torch.bfloat16), (0.1 * rn(C)).to(torch.bfloat16), ru(H, -3.0, -1.0),
                                                -ru(H, 1.0, 16.0), 1.0 + 0.1 * rn(H), norm(DI), norm(), gu, dn))
        self.final_norm = norm()
        hw = exl3.Bits.of(cfg.head_bits or cfg.bits).tile_words
        self.lm_head = lin(d, cfg.vocab_padded, 1.0 / math.sqrt(d), hw, real_n=cfg.vocab)

    def state_view(self, li: int) -> torch.Tensor:
        """The recurrent state pool of layer `li` in canonical order: Mamba2 [slots, H, P, N]; delta-net [slots, Hv, value j, key i] (the
        delta-net pool is stored in the kernel's access order: [warp = j / 16][step][lane = 2 (j % 16) + half][4], i = 64 half + 4 step + e)."""
        pool = self.ssm_pool[li]
        return pool if self.layers[li]["kind"] == "M" else delta_state_canonical(pool)

    def state_bytes(self) -> int:
        return sum(t.numel() * 4 for t in self.conv_pool.values()) + sum(t.numel() * 4 for t in self.ssm_pool.values())

    # ------------------------------------------------------------------ forward
    def _mixer(self, li, L, M, cls, xr_d, xr_a, q, positions, slots, row_seq, ctx_len, block_table, prefill, max_ctx, scale):
        if L["kind"] == "A":
            return super()._mixer(li, L, M, cls, xr_d, xr_a, q, positions, slots, row_seq, ctx_len, block_table, prefill, max_ctx, scale)
        cfg, K = self.cfg, self.K
        seg_s, seg_l, nseg = (prefill["q_start"], prefill["q_len"], prefill["nseq"]) if prefill is not None else (None, None, 0)
        mode = self.ssm_mode if prefill is None else K.SCAN_FINAL
        rec = mode == K.SCAN_RECORD
        if rec and M > self.rec_rows:
            raise ValueError(f"a recorded window of {M} rows exceeds the {self.rec_rows} rows the record buffers hold")
        xbc = self.rec_xbc[li] if rec else self.ssm_xbc
        if L["kind"] in "GK":
            kda = L["kind"] == "K"
            wp = cfg.delta_proj_width(L["kind"])
            s = self._linear(xr_d, L["in_proj"], M, cls, "kda_in" if kda else "gdn_in")
            proj = self.rec_proj[li][:M] if rec else self.ssm_proj[:M * wp].view(M, wp)
            K.finish_store(self.part, s, M, L["in_proj"], proj)
            out = self.ssm_out[:M * cfg.gdn_inner].view(M, cfg.gdn_inner)
            K.gdn_mixer(proj, M, cfg.gdn_k_heads, cfg.gdn_v_heads, 128, row_seq, positions, seg_s, seg_l, nseg, L["conv_w"], L["conv_b"], L["dt_bias"],
                        L["a_neg"], L["norm_w"], cfg.eps, self.conv_pool[li], self.ssm_pool[li], xbc, out, kda=kda, mode=mode, y32=self.ssm_y)
            xr_g = self.xr[:M * cfg.gdn_inner].view(M, cfg.gdn_inner)
            K.norm_rot_in(out, None, cfg.eps, L["out_proj"].suh, xr_g)
            return self._linear(xr_g, L["out_proj"], M, cls, "gdn_out")
        s = self._linear(xr_d, L["in_proj"], M, cls, "in_proj")
        proj = self.rec_proj[li][:M] if rec else self.ssm_proj[:M * cfg.in_proj_width].view(M, cfg.in_proj_width)
        K.finish_store(self.part, s, M, L["in_proj"], proj)
        out = self.ssm_out[:M * cfg.d_inner].view(M, cfg.d_inner)
        K.ssm_mixer(proj, M, cfg.ssm_heads, cfg.ssm_head_dim, cfg.ssm_groups, cfg.ssm_state, row_seq, positions, seg_s, seg_l, nseg, L["conv_w"], L["conv_b"],
                    L["dt_bias"], L["a_neg"], L["d_skip"], L["norm_w"], cfg.eps, self.conv_pool[li], self.ssm_pool[li], xbc, self.ssm_y, out, mode=mode)
        xr_m = self.xr[:M * cfg.d_inner].view(M, cfg.d_inner)
        K.norm_rot_in(out, None, cfg.eps, L["out_proj"].suh, xr_m)
        return self._linear(xr_m, L["out_proj"], M, cls, "out_proj")
