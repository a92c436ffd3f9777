"""Tensor-parallel dense GQA decoder: one shard per GPU, fused compute+collective kernels over NVLink peer memory.

Sharding (Megatron layout; the reference slices output columns at 128-column tiles and replicates what does not divide,
crates/exl3/src/tp.rs:39-123 - here heads and FFN columns are split, o_proj / down_proj are split along K):
  qkv, gate_up, lm_head : column-parallel (input = all-gathered activations, output local)
  o_proj, down_proj     : row-parallel (input local, output reduce-scattered: every rank owns d/R columns of the residual)
Prefill slices, per layer and rank:  GEMM qkv [waits for the gathered input rank by rank] -> finish+RoPE+KV write ->
attention (local heads) -> GEMM o [epilogue pushes tiles to their owner] -> finish_rs (sum, Hadamard, residual, sum of squares
push) -> norm_rot_push (RMSNorm with the all-rank sum, next rotation, all-gather by push) -> GEMM gate_up -> SwiGLU -> GEMM down -> ...
Decode / verify windows (<= 256 rows) are latency-bound, so they use a one-shot all-reduce instead: every rank finishes its own
partial rows (split sum, Hadamard, svh) and pushes them to all ranks, one kernel later each rank adds the R rows in rank order
into a replicated residual stream and normalises / rotates the full row (one NVLink hop per projection instead of three).
No NCCL call is on either path.  `run_phases` exposes the kernels phase by phase so that R shards can be stepped on ONE GPU
(LoopbackGroup) to test the protocol and the numerics.
"""
from __future__ import annotations

import ctypes
import math

import numpy as np
import torch

from ..format import exl3
from ..format.tp import tile_cut
from ..ops import kernels as K
from ..ops import lib as _lib
from ..parallel.symm import ArenaLayout, _GroupBase, check_abi
from .dense import PAGE, DenseConfig, HostLinear, HostWeights, rope_inv_freq


def _cols(l: HostLinear, lo: int, hi: int) -> HostLinear:
    return HostLinear(np.ascontiguousarray(l.trellis[:, lo // 16:hi // 16]), l.suh, np.ascontiguousarray(l.svh[lo:hi]),
                      None if l.bias is None else l.bias[lo:hi], l.codebook)


def _rows(l: HostLinear, lo: int, hi: int) -> HostLinear:
    return HostLinear(np.ascontiguousarray(l.trellis[lo // 16:hi // 16]), np.ascontiguousarray(l.suh[lo:hi]), l.svh, l.bias, l.codebook)


def _cat_cols(parts) -> HostLinear:
    return HostLinear(np.concatenate([p.trellis for p in parts], axis=1), parts[0].suh, np.concatenate([p.svh for p in parts]),
                      None if parts[0].bias is None else np.concatenate([p.bias for p in parts]), parts[0].codebook)


def shard_weights(w: HostWeights, rank: int, ranks: int) -> dict:
    """Slices of a full model for one rank (whole 128-column tiles / 128-row Hadamard blocks only)."""
    cfg = w.cfg
    hd, F = cfg.head_dim, cfg.ffn_padded
    if cfg.n_q % ranks or cfg.n_kv % ranks or (cfg.d_model // ranks) % 128 or (F // ranks) % 128 or F % ranks:
        raise ValueError(f"{cfg.name}: heads {cfg.n_q}/{cfg.n_kv}, d {cfg.d_model}, ffn {F} do not split over {ranks} ranks at 128-column tiles")
    ql, kl = cfg.n_q // ranks * hd, cfg.n_kv // ranks * hd
    if ql % 128 or kl % 128:
        raise ValueError("per-rank q / kv widths must be multiples of 128")
    Q, KV = cfg.n_q * hd, cfg.n_kv * hd
    fl = F // ranks
    layers = []
    for L in w.layers:
        qkv = _cat_cols([_cols(L.qkv, rank * ql, (rank + 1) * ql), _cols(L.qkv, Q + rank * kl, Q + (rank + 1) * kl),
                         _cols(L.qkv, Q + KV + rank * kl, Q + KV + (rank + 1) * kl)])
        gu = _cat_cols([_cols(L.gate_up, rank * fl, (rank + 1) * fl), _cols(L.gate_up, F + rank * fl, F + (rank + 1) * fl)])
        layers.append(dict(attn_norm=L.attn_norm, ffn_norm=L.ffn_norm, qkv=qkv, o=_rows(L.o, rank * ql, (rank + 1) * ql), gate_up=gu,
                           down=_rows(L.down, rank * fl, (rank + 1) * fl), q_norm=L.q_norm, k_norm=L.k_norm))
    s0, s1 = tile_cut(cfg.vocab_padded // 128, rank, ranks)
    return dict(embed=w.embed, layers=layers, final_norm=w.final_norm, lm_head=_cols(w.lm_head, s0 * 128, s1 * 128), vocab_lo=s0 * 128, vocab_hi=s1 * 128)


class DenseTPShard:
    """One rank of the tensor-parallel model."""

    def __init__(self, cfg: DenseConfig, group: _GroupBase, rank: int, num_pages: int, max_rows: int, max_seqs: int, max_blocks_per_seq: int,
                 weights: dict | None = None, device="cuda", seed: int = 0, kv_dtype: str = "bf16", collective: str = "fused"):
        """`collective`: "fused" (peer-memory kernels, the product) or "nccl" (the baseline for comparison: decode windows finish their partial
        rows locally and call NCCL all-reduce on the f32 rows; prefill slices are unchanged)."""
        check_abi()
        if collective not in ("fused", "nccl"):
            raise ValueError(collective)
        self.collective = collective
        self.ar_local = None
        self.cfg, self.g, self.rank, self.R, self.device = cfg, group, rank, group.ranks, device
        R = self.R
        self.nq, self.nkv = cfg.n_q // R, cfg.n_kv // R
        self.d, self.n_own, self.col0 = cfg.d_model, cfg.d_model // R, rank * (cfg.d_model // R)
        self.F = cfg.ffn_padded // R
        self.max_rows, self.num_pages, self.max_blocks = max_rows, num_pages, max_blocks_per_seq
        if weights is not None:
            self._load(weights)
        else:
            self._random(seed)
        self.inv_freq = torch.from_numpy(rope_inv_freq(cfg)).to(device)
        hd = cfg.head_dim
        self.kv_fp8 = kv_dtype == "fp8"
        cdt = torch.uint8 if self.kv_fp8 else torch.bfloat16
        self.k_cache = [torch.zeros(num_pages, self.nkv, PAGE, hd, dtype=cdt, device=device) for _ in range(cfg.n_layers)]
        self.v_cache = [torch.zeros(num_pages, self.nkv, PAGE, hd, dtype=cdt, device=device) for _ in range(cfg.n_layers)]
        self.kv_scale = torch.ones(cfg.n_layers, 2, self.nkv, dtype=torch.float32, device=device) if self.kv_fp8 else None
        self.kv_amax = None
        self.tk = [K.KvTensorMap(c) for c in self.k_cache]
        self.tv = [K.KvTensorMap(c) for c in self.v_cache]
        self.status = K.new_status(device)
        self.splits = {}
        part = 0
        shapes = dict(qkv=(cfg.d_model, (self.nq + 2 * self.nkv) * hd), o=(self.nq * hd, cfg.d_model), gate_up=(cfg.d_model, 2 * self.F),
                      down=(self.F, cfg.d_model), lm_head=(cfg.d_model, self.lm_head.N))
        for cls, rows in (("decode", min(max_rows, 256)), ("prefill", max_rows)):
            for name, (k, n) in shapes.items():
                s = K.plan_splits(k, n, cls == "decode")
                self.splits[(cls, name)] = s
                if name in ("qkv", "gate_up", "lm_head") or cls == "decode":      # decode windows keep o / down partials local too
                    part = max(part, s * (rows if name != "lm_head" else min(rows, 256)) * n)
        self.part = torch.empty(part, dtype=torch.float32, device=device)
        self.h = torch.empty(max_rows, cfg.d_model, dtype=torch.bfloat16, device=device)
        self.q = torch.empty(max_rows, self.nq * hd, dtype=torch.bfloat16, device=device)
        self.xr_a = torch.empty(max_rows * self.nq * hd, dtype=torch.float16, device=device)
        self.xr_f = torch.empty(max_rows * self.F, dtype=torch.float16, device=device)
        self.xr0 = torch.empty(max_rows * cfg.d_model, dtype=torch.float16, device=device)      # layer-0 input (computed locally)
        self.xr_d = torch.empty(min(max_rows, 256) * cfg.d_model, dtype=torch.float16, device=device)   # decode windows: full-width rotated input
        self.attn_out = torch.empty(max_rows, self.nq * hd, dtype=torch.bfloat16, device=device)
        self.logits = torch.empty(min(max_rows, 256), self.lm_head.N, dtype=torch.float32, device=device)
        self.topk_scratch = K.topk_scratch(min(max_rows, 256), self.lm_head.N, 64, device)
        self.loc_ids = torch.empty(256 * 64, dtype=torch.int32, device=device)
        self.loc_vals = torch.empty(256 * 64, dtype=torch.float32, device=device)
        self.cand_ids = torch.empty(256 * 64, dtype=torch.int32, device=device)      # merged result (leader)
        self.cand_vals = torch.empty(256 * 64, dtype=torch.float32, device=device)
        self.attn_scratch = K.attn_decode_scratch(min(max_rows, 256), self.nq, hd, max_blocks_per_seq * PAGE, device)
        self.attn_plan = K.attn_plan_buffer(device)
        self.max_ctx_alloc = max_blocks_per_seq * PAGE

    @staticmethod
    def plane_elems(cfg: DenseConfig, ranks: int, max_rows: int) -> int:
        """Room one source rank's reduce-scatter planes need (max over the decode and prefill row classes and the two sites)."""
        n_own = cfg.d_model // ranks
        hd = cfg.head_dim
        worst = 0
        for decode, rows in ((True, min(max_rows, 256)), (False, max_rows)):
            for k in (cfg.n_q // ranks * hd, cfg.ffn_padded // ranks):
                worst = max(worst, K.plan_splits(k, cfg.d_model, decode) * rows * n_own)
        return worst

    @staticmethod
    def layout(cfg: DenseConfig, ranks: int, max_rows: int) -> ArenaLayout:
        return ArenaLayout(ranks, max_rows, DenseTPShard.plane_elems(cfg, ranks, max_rows), cfg.d_model, cfg.d_model // ranks)

    # ------------------------------------------------------------------ weights
    def _load(self, w: dict) -> None:
        dev = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(device=self.device, dtype=dt)  # noqa: E731
        up = lambda l: K.Exl3Weight.from_numpy(l.trellis, l.suh, l.svh, l.bias, l.codebook, self.device)  # noqa: E731
        self.embed = dev(w["embed"], torch.bfloat16)
        self.layers = [dict(attn_norm=dev(L["attn_norm"], torch.bfloat16), ffn_norm=dev(L["ffn_norm"], torch.bfloat16), qkv=up(L["qkv"]), o=up(L["o"]),
                            gate_up=up(L["gate_up"]), down=up(L["down"]), q_norm=None if L["q_norm"] is None else dev(L["q_norm"], torch.bfloat16),
                            k_norm=None if L["k_norm"] is None else dev(L["k_norm"], torch.bfloat16)) for L in w["layers"]]
        self.final_norm = dev(w["final_norm"], torch.bfloat16)
        self.lm_head = up(w["lm_head"])
        self.vocab_lo, self.vocab_hi = w["vocab_lo"], w["vocab_hi"]

    def _random(self, seed: int) -> None:
        """Random-init shard generated on the device (benchmarks).  Replicated tensors (embedding, norms, input scales of the
        column-parallel layers) come from a seed shared by all ranks; the trellis shards from a per-rank seed."""
        cfg, dev = self.cfg, self.device
        shared = torch.Generator(device=dev).manual_seed(seed)
        own = torch.Generator(device=dev).manual_seed(seed * 1000 + 17 + self.rank)
        tw = exl3.Bits.of(cfg.bits).tile_words
        hd, d = cfg.head_dim, cfg.d_model
        sg = lambda m, g: (torch.randint(0, 2, (m,), device=dev, generator=g) * 2 - 1).to(torch.float16)  # noqa: E731

        def lin(k, n, scale, suh):
            tr = torch.randint(-32768, 32768, (k // 16, n // 16, tw), dtype=torch.int16, device=dev, generator=own)
            return K.Exl3Weight(tr, suh, (sg(n, own) * scale).to(torch.float16), None, cfg.codebook)
        norm = lambda: (1.0 + 0.1 * torch.randn(d, device=dev, generator=shared)).to(torch.bfloat16)  # noqa: E731
        self.embed = torch.randn(cfg.vocab, d, device=dev, generator=shared).to(torch.bfloat16)
        self.layers = []
        for _ in range(cfg.n_layers):
            an, fn = norm(), norm()
            su_qkv, su_gu = sg(d, shared), sg(d, shared)
            self.layers.append(dict(attn_norm=an, ffn_norm=fn, qkv=lin(d, (self.nq + 2 * self.nkv) * hd, 1 / math.sqrt(d), su_qkv),
                                    o=lin(self.nq * hd, d, 0.5 / math.sqrt(cfg.n_q * hd), sg(self.nq * hd, own)),
                                    gate_up=lin(d, 2 * self.F, 1 / math.sqrt(d), su_gu),
                                    down=lin(self.F, d, 0.5 / math.sqrt(cfg.ffn_padded), sg(self.F, own)), q_norm=None, k_norm=None))
        self.final_norm = norm()
        s0, s1 = tile_cut(cfg.vocab_padded // 128, self.rank, self.R)
        self.vocab_lo, self.vocab_hi = s0 * 128, s1 * 128
        self.lm_head = lin(d, (s1 - s0) * 128, 1 / math.sqrt(d), sg(d, shared))

    # ------------------------------------------------------------------ kernels with TP descriptors
    def _gemm(self, xr, w, part_ptr, splits, desc):
        rows, k = xr.shape
        L = _lib.load()
        _lib.check(L.rx_exl3_gemm_b4_tp(xr.data_ptr(), rows, k, w.trellis.data_ptr(), w.N, K.CB_ID[w.codebook], part_ptr, splits,
                                        self.status.data_ptr(), _lib.stream_ptr(), ctypes.byref(desc)), "rx_exl3_gemm_b4_tp")
        _lib.count()

    def phases(self, ids, positions, slots, row_seq, ctx_len, block_table, prefill=None, max_ctx=None, want_logits=True, logit_rows=None,
               cand_count=None, leader=0, tree=None):
        """Generator of closures, one per phase; calling them in order runs this rank's forward.  Between two phases every
        cross-rank dependency points backwards, so a loopback group may interleave the ranks phase by phase."""
        cfg, g, r, R = self.cfg, self.g, self.rank, self.R
        if cfg.bits != 4.0:
            raise NotImplementedError("the tensor-parallel path uses the 4.0 bpw tensor-memory GEMM")
        M = ids.shape[0]
        cls = "decode" if prefill is None else "prefill"
        hd, d, F = cfg.head_dim, self.d, self.F
        h = self.h[:M]
        q = self.q[:M]
        xr_a = self.xr_a[:M * self.nq * hd].view(M, self.nq * hd)
        xr_f = self.xr_f[:M * F].view(M, F)
        xr0 = self.xr0[:M * d].view(M, d)
        scale = 1.0 / math.sqrt(hd)
        Lib = _lib.load()
        sp = self.splits
        nl = len(self.layers)

        def p_start():
            _lib.check(Lib.rx_tp_bump_epoch(g.epoch_ptr(r), _lib.stream_ptr()), "rx_tp_bump_epoch")
            if prefill is None:
                K.attn_plan(row_seq, ctx_len, self.nq, self.nkv, getattr(self, "window_seq_rows", 1), self.attn_plan,
                            tree_base=None if tree is None else tree[0])
            K.embed(ids, self.embed, h)
            K.norm_rot_in(h, self.layers[0]["attn_norm"], cfg.eps, self.layers[0]["qkv"].suh, xr0)
        yield p_start

        if prefill is None:
            yield from self._window_phases(M, positions, slots, row_seq, ctx_len, block_table, max_ctx, h, q, xr_a, xr_f, xr0, tree)
        else:
            yield from self._prefill_phases(M, positions, slots, block_table, prefill, h, q, xr_a, xr_f, xr0)
        yield from self._head_phases(M, want_logits, logit_rows, cand_count, leader, prefill is None)

    def supports_trees(self) -> bool:
        return True

    def _kv_ptr_table(self):
        if getattr(self, "_kv_ptrs", None) is None:
            self._kv_ptrs = torch.tensor([c.data_ptr() for kv in zip(self.k_cache, self.v_cache) for c in kv], dtype=torch.int64, device=self.device)
        return self._kv_ptrs

    def move_kv_rows(self, moves, n_moves: int) -> None:
        """(source slot, destination slot, rows) copies over this rank's K and V caches of every layer (see DenseGPU.move_kv_rows)."""
        c = self.k_cache[0]
        K.kv_move_rows(self._kv_ptr_table(), c.shape[-1] * c.element_size(), self.nkv, moves, n_moves)

    def _window_phases(self, M, positions, slots, row_seq, ctx_len, block_table, max_ctx, h, q, xr_a, xr_f, xr0, tree=None):
        """Decode / verify windows (rows <= 256): one-shot all-reduce after o_proj and down_proj, residual stream replicated.
        tree = (tree_base, vbt, row copies, count): a window of draft trees (see DenseGPU.forward_phases); the slots, private tables and copies
        are the same on every rank, each rank applies them to its own KV heads."""
        cfg, g, r, R = self.cfg, self.g, self.rank, self.R
        from ..parallel.symm import AR_ROWS
        hd, d = cfg.head_dim, self.d
        scale = 1.0 / math.sqrt(hd)
        Lib = _lib.load()
        sp = self.splits
        nl = len(self.layers)
        if M > AR_ROWS:
            raise ValueError(f"a window of {M} rows exceeds the {AR_ROWS}-row all-reduce slots")
        xr_d = self.xr_d[:M * d].view(M, d)
        none = ctypes.c_void_p(0)

        def chain_nccl(x_part, s, w, norm_w, suh_next):
            """Comparison path: finish locally, NCCL all-reduce of the f32 rows, then the same residual / norm / rotate kernel on one slot."""
            import torch.distributed as dist
            if self.ar_local is None:
                self.ar_local = torch.zeros(AR_ROWS, d, dtype=torch.float32, device=self.device)

            def p_push():
                buf = self.ar_local[:M]
                K.finish_store(x_part, s, M, w, buf)
                if R > 1 and w.bias is not None and r != 0:
                    buf.sub_(w.bias)                   # the bias counts once
                dist.all_reduce(buf)

            def p_sum():
                _lib.check(Lib.rx_tp_allsum_add_norm_rot(self.ar_local.data_ptr(), None, 1, AR_ROWS, None, 0, M, d, h.data_ptr(), norm_w.data_ptr(),
                                                         cfg.eps, suh_next.data_ptr(), xr_d.data_ptr(), self.status.data_ptr(), _lib.stream_ptr(), None),
                           "rx_tp_allsum_add_norm_rot")
                _lib.count()
            return p_push, p_sum

        def chain(x_part, s, w, parity, use, norm_w, suh_next):
            """Two phases: push this rank's finished partial rows to every rank; sum all ranks' rows into the residual, norm, rotate."""
            if self.collective == "nccl":
                return chain_nccl(x_part, s, w, norm_w, suh_next)

            def p_push():
                _lib.check(Lib.rx_tp_finish_bcast_mm(x_part.data_ptr(), s, M, d, w.svh.data_ptr(), None if (w.bias is None or r != 0) else w.bias.data_ptr(),
                                                     ctypes.byref(g.bcast(r, parity, use)), _lib.stream_ptr(), g.mm_local(parity) or None),
                           "rx_tp_finish_bcast_mm")
                _lib.count()

            def p_sum():
                # with an NVLS buffer bound (g.mm_mc): windows above the packet size read the sum over ranks from the switch
                _lib.check(Lib.rx_tp_allsum_add_norm_rot_mm(g.ar_ptr(r, parity), g.ar_flag_ptr(r, parity), R, AR_ROWS, g.epoch_ptr(r), use, M, d,
                                                            h.data_ptr(), norm_w.data_ptr(), cfg.eps, suh_next.data_ptr(), xr_d.data_ptr(),
                                                            self.status.data_ptr(), _lib.stream_ptr(), None, g.mm_mc(parity) or None),
                           "rx_tp_allsum_add_norm_rot_mm")
                _lib.count()
            return p_push, p_sum

        for li, L in enumerate(self.layers):
            u_o, u_d = 2 * li + 1, 2 * li + 2

            def p_attn(li=li, L=L):
                x_in = xr0 if li == 0 else xr_d
                s = sp[("decode", "qkv")]
                K.exl3_gemm(x_in, L["qkv"], self.part, s, self.status)
                ksc = self.kv_scale[li] if self.kv_fp8 else None
                K.finish_qkv_rope(self.part, s, M, self.nq, self.nkv, hd, L["qkv"], L["q_norm"], L["k_norm"], cfg.eps, positions, self.inv_freq,
                                  slots, q, self.k_cache[li], self.v_cache[li], ksc)
                if tree is not None:
                    c = self.k_cache[li]
                    K.kv_move_rows(self._kv_ptr_table()[2 * li:2 * li + 2], c.shape[-1] * c.element_size(), self.nkv, tree[2], tree[3])
                K.attn_decode(self.tk[li], self.tv[li], q, block_table, row_seq, ctx_len, self.attn_scratch, self.nq, self.nkv, hd,
                              max_ctx or self.max_ctx_alloc, scale, L["o"].suh, xr_a, None, self.status, ksc,
                              max_seq_rows=getattr(self, "window_seq_rows", 1), plan=self.attn_plan, vbt=None if tree is None else tree[1])
                K.exl3_gemm(xr_a, L["o"], self.part, sp[("decode", "o")], self.status)
            yield p_attn
            a, b = chain(self.part, sp[("decode", "o")], L["o"], 0, u_o, L["ffn_norm"], L["gate_up"].suh)
            yield a
            yield b

            def p_mlp(L=L):
                s = sp[("decode", "gate_up")]
                K.exl3_gemm(xr_d, L["gate_up"], self.part, s, self.status)
                K.finish_swiglu_rot(self.part, s, M, L["gate_up"], L["down"].suh, xr_f)
                K.exl3_gemm(xr_f, L["down"], self.part, sp[("decode", "down")], self.status)
            yield p_mlp
            nw, su = (self.layers[li + 1]["attn_norm"], self.layers[li + 1]["qkv"].suh) if li + 1 < nl else (self.final_norm, self.lm_head.suh)
            a, b = chain(self.part, sp[("decode", "down")], L["down"], 1, u_d, nw, su)
            yield a
            yield b

    def _prefill_phases(self, M, positions, slots, block_table, prefill, h, q, xr_a, xr_f, xr0):
        """Prefill slices (many rows): reduce-scatter in the GEMM epilogue, all-gather feeding the next GEMM, residual stream sharded."""
        cfg, g, r, R = self.cfg, self.g, self.rank, self.R
        cls = "prefill"
        hd, d = cfg.head_dim, self.d
        scale = 1.0 / math.sqrt(hd)
        Lib = _lib.load()
        sp = self.splits
        nl = len(self.layers)
        for li, L in enumerate(self.layers):
            u_o, u_d = 2 * li + 1, 2 * li + 2

            def p_attn(li=li, L=L, u_o=u_o):
                x_in = xr0 if li == 0 else g.xr_view(r, 1, M)
                desc = g.gemm_ag(r, 1, 2 * li, d)             # ticket of the previous layer's down-projection chain
                if li == 0:
                    desc.in_flag = None
                s = sp[(cls, "qkv")]
                self._gemm(x_in, L["qkv"], self.part.data_ptr(), s, desc)
                ksc = self.kv_scale[li] if self.kv_fp8 else None
                K.finish_qkv_rope(self.part, s, M, self.nq, self.nkv, hd, L["qkv"], L["q_norm"], L["k_norm"], cfg.eps, positions, self.inv_freq,
                                  slots, q, self.k_cache[li], self.v_cache[li], ksc, None if self.kv_amax is None else self.kv_amax[li])
                ao = self.attn_out[:M]
                K.attn_prefill(self.tk[li], self.tv[li], q, block_table, prefill["seq_ids"], prefill["q_start"], prefill["q_len"],
                               prefill["pos0"], ao, prefill["nseq"], prefill["max_qlen"], self.nq, self.nkv, hd, scale, self.status, ksc)
                K.norm_rot_in(ao, None, cfg.eps, L["o"].suh, xr_a)
                so = sp[(cls, "o")]
                self._gemm(xr_a, L["o"], g.part_ptr(r, 0), so, g.gemm_rs(r, 0, u_o, so, M))
            yield p_attn

            def p_fin_o(L=L, u_o=u_o):
                so = sp[(cls, "o")]
                svh = L["o"].svh[self.col0:self.col0 + self.n_own]
                _lib.check(Lib.rx_tp_finish_rs(g.part_ptr(r, 0), so, M, self.n_own, d, self.col0, svh.data_ptr(), None, h.data_ptr(),
                                               self.status.data_ptr(), ctypes.byref(g.finish(r, 0, 0, u_o)), _lib.stream_ptr()), "rx_tp_finish_rs")
                _lib.count()
            yield p_fin_o

            def p_push_o(L=L, u_o=u_o):
                _lib.check(Lib.rx_tp_norm_rot_push(h.data_ptr(), M, self.n_own, d, self.col0, L["ffn_norm"].data_ptr(), cfg.eps,
                                                   L["gate_up"].suh.data_ptr(), self.status.data_ptr(), ctypes.byref(g.push(r, 0, u_o)),
                                                   _lib.stream_ptr()), "rx_tp_norm_rot_push")
                _lib.count()
            yield p_push_o

            def p_mlp(L=L, u_o=u_o, u_d=u_d):
                s = sp[(cls, "gate_up")]
                self._gemm(g.xr_view(r, 0, M), L["gate_up"], self.part.data_ptr(), s, g.gemm_ag(r, 0, u_o, d))
                K.finish_swiglu_rot(self.part, s, M, L["gate_up"], L["down"].suh, xr_f)
                sd = sp[(cls, "down")]
                self._gemm(xr_f, L["down"], g.part_ptr(r, 1), sd, g.gemm_rs(r, 1, u_d, sd, M))
            yield p_mlp

            def p_fin_d(L=L, u_d=u_d):
                sd = sp[(cls, "down")]
                svh = L["down"].svh[self.col0:self.col0 + self.n_own]
                _lib.check(Lib.rx_tp_finish_rs(g.part_ptr(r, 1), sd, M, self.n_own, d, self.col0, svh.data_ptr(), None, h.data_ptr(),
                                               self.status.data_ptr(), ctypes.byref(g.finish(r, 1, 1, u_d)), _lib.stream_ptr()), "rx_tp_finish_rs")
                _lib.count()
            yield p_fin_d

            def p_push_d(li=li, u_d=u_d):
                nw, su = (self.layers[li + 1]["attn_norm"], self.layers[li + 1]["qkv"].suh) if li + 1 < nl else (self.final_norm, self.lm_head.suh)
                _lib.check(Lib.rx_tp_norm_rot_push(h.data_ptr(), M, self.n_own, d, self.col0, nw.data_ptr(), cfg.eps, su.data_ptr(),
                                                   self.status.data_ptr(), ctypes.byref(g.push(r, 1, u_d)), _lib.stream_ptr()), "rx_tp_norm_rot_push")
                _lib.count()
            yield p_push_d

    def _head_phases(self, M, want_logits, logit_rows, cand_count, leader, window):
        cfg, g, r, R = self.cfg, self.g, self.rank, self.R
        d = self.d
        Lib = _lib.load()
        sp = self.splits
        nl = len(self.layers)

        def p_head():
            if not want_logits:
                return None
            x = g.xr_view(r, 1, M) if not window else self.xr_d[:M * d].view(M, d)
            desc = g.gemm_ag(r, 1, 2 * nl, d)
            if window:
                desc.in_flag = None
                if logit_rows is not None:
                    x = x.index_select(0, logit_rows).contiguous()
            elif logit_rows is not None:
                # a library gather reads the pushed buffer: hold the stream until every rank's slice has landed
                _lib.check(Lib.rx_tp_wait_flags(desc.in_flag, R, g.epoch_ptr(r), 2 * nl, self.status.data_ptr(), _lib.stream_ptr()), "rx_tp_wait_flags")
                x = x.index_select(0, logit_rows).contiguous()
                desc.in_flag = None
            Rw = x.shape[0]
            s = sp[("decode", "lm_head")]
            self._gemm(x, self.lm_head, self.part.data_ptr(), s, desc)
            out = self.logits[:Rw]
            K.finish_store(self.part, s, Rw, self.lm_head, out)
            self.last_logits = out
            return out
        yield p_head

        if want_logits and cand_count is not None:
            Rw = M if logit_rows is None else int(logit_rows.shape[0])
            u_c = 2 * nl + 1

            def p_cand_push():
                out = self.last_logits
                if self.vocab_hi > cfg.vocab:                      # padded vocabulary columns never become candidates
                    out[:, max(0, cfg.vocab - self.vocab_lo):] = float("-inf")
                K.topk(out, cand_count, self.topk_scratch, self.loc_ids[:Rw * cand_count].view(Rw, cand_count),
                       self.loc_vals[:Rw * cand_count].view(Rw, cand_count))
                _lib.check(Lib.rx_tp_cand_push(self.loc_ids.data_ptr(), self.loc_vals.data_ptr(), Rw, cand_count,
                                               ctypes.byref(g.cand(r, leader, u_c, self.vocab_lo)), _lib.stream_ptr()), "rx_tp_cand_push")
                _lib.count()
            yield p_cand_push

            def p_cand_merge():
                if r != leader:
                    return None
                from ..parallel.symm import CAND_ROWS
                La, b = g.layout, g.base(r, r)
                _lib.check(Lib.rx_tp_cand_merge(b + La.cand_ids, b + La.cand_vals, b + La.cand_flag, R, Rw, cand_count, CAND_ROWS, g.epoch_ptr(r), u_c,
                                                self.cand_ids.data_ptr(), self.cand_vals.data_ptr(), self.status.data_ptr(), _lib.stream_ptr()),
                           "rx_tp_cand_merge")
                _lib.count()
                return self.cand_ids[:Rw * cand_count].view(Rw, cand_count), self.cand_vals[:Rw * cand_count].view(Rw, cand_count)
            yield p_cand_merge

    def calibrate_kv(self, tokens, passes: int = 2, headroom: float = 1.25) -> None:
        """FP8 cache: per-head scales from a calibration prefill (see DenseGPU.calibrate_kv).  Every rank of the group calls this with the same
        tokens at the same time (the forward contains the group's collectives)."""
        if not self.kv_fp8:
            return
        T = len(tokens)
        dev = self.device
        nb = (T + PAGE - 1) // PAGE
        bt = torch.zeros(8, max(nb, 1), dtype=torch.int32, device=dev)
        bt[0, :nb] = torch.arange(nb, dtype=torch.int32, device=dev)
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)  # noqa: E731
        pos = list(range(T))
        pf = dict(seq_ids=i32([0]), q_start=i32([0]), q_len=i32([T]), pos0=i32([0]), nseq=1, max_qlen=T)
        for _ in range(passes):
            self.kv_amax = torch.zeros_like(self.kv_scale)
            self.forward(i32(list(tokens)), i32(pos), i32(pos), i32([0] * T), i32([p + 1 for p in pos]), bt, prefill=pf, want_logits=False)
            torch.cuda.synchronize()
            self.kv_scale.copy_(torch.clamp(self.kv_amax, min=1e-4) * (headroom / 448.0))
        self.kv_amax = None

    def forward(self, *a, **kw):
        out = None
        for p in self.phases(*a, **kw):
            out = p()
        return out
