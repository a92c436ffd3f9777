"""Backend over the sm_100a dense executor: slots, paged KV bookkeeping, pinned-host staging of the per-step row
arrays, CUDA-graph replay of decode windows, device top-k with a small device->host read per step.

Only this module touches the GPU on behalf of the engine (one engine thread owns the CUDA context, as in the
reference's runtime, crates/server/src/runtime.rs:603).  Per step the host uploads five small int32 arrays
(ids, positions, KV slots, row->sequence, context lengths) from pinned memory and reads back rows x count candidate
(id, value) pairs; the full logits never leave the device (reference crates/model/src/forward.rs:1519-1552).
"""
from __future__ import annotations

import numpy as np
import torch

from ..models.dense import PAGE, DenseGPU
from ..sched import BlockPool
from .backend import Backend, BackendError, RowOutput

CTX_BUCKET = 2048   # decode graphs are captured per (rows, candidate count, context bucket)


class DenseGpuBackend(Backend):
    name = "cuda"

    def __init__(self, model: DenseGPU, max_slots: int | None = None, use_graphs: bool = True, self_draft: bool = False, mtp_draft: bool = False):
        """`self_draft`: offer drafts from the model's first `cfg.draft_layers` layers plus the shared final norm and head (the draft
        shares the target's KV cache for those layers, so it needs no state of its own).
        `mtp_draft`: offer drafts from the model's multi-token-prediction block (config.mtp).  The block's KV rows lag the trunk by one
        position: whenever the trunk runs rows whose tokens are known, the block runs the rows one position earlier (hidden of position
        i, token i + 1), reading the trunk's final residual rows; the last window's rows are kept per slot so that the row before the next
        window is at hand whatever number of drafts was accepted.  Draft j chains the block on its own output hidden."""
        self.m = model
        self.self_draft = bool(self_draft and getattr(model.cfg, "draft_layers", 0) > 0)
        self.mtp_draft = bool(mtp_draft and getattr(model, "mtp", None) is not None)
        if mtp_draft and not self.mtp_draft:
            raise ValueError("mtp_draft needs a model with a multi-token-prediction block (config.mtp)")
        self.cfg = model.cfg
        self.vocab_size = model.cfg.vocab
        self.max_slots = max_slots or model.max_seqs
        self.max_rows = min(256, model.max_rows)
        # paged experts read the router's picks on the host in every layer: nothing there can be captured
        self.use_graphs = use_graphs and getattr(model, "paged", None) is None
        self.pool = BlockPool(model.num_pages, PAGE)
        self.len = [0] * self.max_slots            # committed tokens per slot
        self.pages = [[] for _ in range(self.max_slots)]
        self.pending = [0] * self.max_slots        # rows of the last window
        dev = model.device
        R = model.max_rows
        self.h_rows = torch.zeros(5, R, dtype=torch.int32).pin_memory()
        self.d_rows = torch.zeros(5, R, dtype=torch.int32, device=dev)
        self.h_bt = torch.zeros(self.max_slots, model.max_blocks, dtype=torch.int32).pin_memory()
        self.d_bt = torch.zeros(self.max_slots, model.max_blocks, dtype=torch.int32, device=dev)
        self.bt_dirty = True
        self.bt_dirty_slots = set(range(self.max_slots))
        self.h_pf = torch.zeros(4, self.max_slots, dtype=torch.int32).pin_memory()
        self.d_pf = torch.zeros(4, self.max_slots, dtype=torch.int32, device=dev)
        self.h_cand_ids = torch.zeros(256, 64, dtype=torch.int32).pin_memory()
        self.h_cand_vals = torch.zeros(256, 64, dtype=torch.float32).pin_memory()
        self.h_status = torch.zeros(8, dtype=torch.int32).pin_memory()
        self.graphs = {}
        self.draft_graphs = {}
        self.draft_steps = 0
        self.DK = 8                                            # most chained drafts one ask may get
        if self.mtp_draft:
            d_model = model.cfg.d_model
            self.MTP_W = 16                                    # trunk rows kept per slot (a window has at most 1 + DK rows)
            NS = self.max_slots * self.MTP_W
            self.mtp_src = torch.zeros(NS + R, d_model, dtype=torch.bfloat16, device=dev)     # [kept rows of every slot | this call's trunk rows]
            self.mtp_in = torch.zeros(R, d_model, dtype=torch.bfloat16, device=dev)
            self.mtp_chain = torch.zeros(self.max_slots, d_model, dtype=torch.bfloat16, device=dev)
            self.mtp_p0 = [-1] * self.max_slots                # first position of the slot's kept rows (-1: none)
            self.mtp_n = [0] * self.max_slots
            self.h_mtp = torch.zeros(6, R, dtype=torch.int32).pin_memory()
            self.d_mtp = torch.zeros(6, R, dtype=torch.int32, device=dev)
            self.h_keep = torch.zeros(2, R, dtype=torch.int64).pin_memory()
            self.d_keep = torch.zeros(2, R, dtype=torch.int64, device=dev)
            self.mtp_rows = 0
        if self.self_draft or self.mtp_draft:
            self.h_draft = torch.zeros(self.DK, 5, self.max_slots, dtype=torch.int32).pin_memory()
            self.d_draft = torch.zeros(self.DK, 5, self.max_slots, dtype=torch.int32, device=dev)
            self.d_draft_ids = torch.zeros(self.DK, self.max_slots, dtype=torch.int32, device=dev)
            self.d_draft_vals = torch.zeros(self.DK, self.max_slots, dtype=torch.float32, device=dev)
            self.h_draft_ids = torch.zeros(self.DK, self.max_slots, dtype=torch.int32).pin_memory()
        # tree windows: per row the anchor's position and the private page table; the per-layer row copies; the accepted paths' row copies
        from ..ops import kernels as _K
        self.VBT_W = _K.attn_vbt_width()
        self.h_tree_base = torch.zeros(R, dtype=torch.int32).pin_memory()
        self.d_tree_base = torch.zeros(R, dtype=torch.int32, device=dev)
        self.h_vbt = torch.zeros(R, self.VBT_W, dtype=torch.int32).pin_memory()
        self.d_vbt = torch.zeros(R, self.VBT_W, dtype=torch.int32, device=dev)
        self.h_spread = torch.zeros(4096, 3, dtype=torch.int32).pin_memory()
        self.d_spread = torch.zeros(4096, 3, dtype=torch.int32, device=dev)
        self.h_moves = torch.zeros(256, 3, dtype=torch.int32).pin_memory()
        self.d_moves = torch.zeros(256, 3, dtype=torch.int32, device=dev)
        self.moves = []                                        # (source slot, destination slot, rows) not yet applied on the device
        self.tree_p0 = [0] * self.max_slots
        self.tree_parents = [None] * self.max_slots
        self.tree_slots = [None] * self.max_slots              # slot of each row of the slot's last tree window
        self.tree_priv = [[] for _ in range(self.max_slots)]   # private pages of the slot's last tree window
        self._tree_n = 0                                       # > 0 while a tree window runs: row copies per layer (padded)
        self.tree_windows = 0
        self.tree_moves = 0
        self.tree_copies = 0
        self.LAT_K = 4                                         # candidates per level the self-draft chain offers (its lattice)
        if self.self_draft:
            self.d_lat_ids = torch.zeros(self.DK, self.max_slots, self.LAT_K, dtype=torch.int32, device=dev)
            self.d_lat_vals = torch.zeros(self.DK, self.max_slots, self.LAT_K, dtype=torch.float32, device=dev)
            self.h_lat_ids = torch.zeros(self.DK, self.max_slots, self.LAT_K, dtype=torch.int32).pin_memory()
            self.h_lat_vals = torch.zeros(self.DK, self.max_slots, self.LAT_K, dtype=torch.float32).pin_memory()
        # image prompts: per slot the MediaInputs of the prompt in flight (embeddings on the device) and what decode rows add to their position
        self.media = [None] * self.max_slots
        self.rope_delta = [0] * self.max_slots
        self.media_rows = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.graph_replays = 0
        self.graph_captures = 0
        self.graph_kernels = {}     # graph key -> kernels launched per replay
        self.replayed_kernels = 0
        self._err = None
        # The pinned staging arrays are read by asynchronous copies queued behind earlier kernels.  An event recorded after the last
        # such copy is waited for before the host writes any of them again (a prefill slice that returns no candidates ends without
        # a stream synchronisation, so the next slice's fill could otherwise overwrite rows the copy engine has not fetched yet).
        self._staged = torch.cuda.Event()
        self._staged_pending = False

    # ------------------------------------------------------------------ staging
    def _host_writable(self) -> None:
        """Blocks until the device has taken every upload issued so far from the pinned staging arrays."""
        if self._staged_pending:
            self._staged.synchronize()
            self._staged_pending = False

    def _uploaded(self) -> None:
        self._staged.record()
        self._staged_pending = True

    # ------------------------------------------------------------------ pages
    def _ensure(self, slot: int, tokens: int) -> None:
        need = self.pool.blocks_for(tokens) - len(self.pages[slot])
        if need <= 0:
            return
        if len(self.pages[slot]) + need > self.m.max_blocks:
            raise BackendError(f"slot {slot}: {tokens} tokens exceed the {self.m.max_blocks * PAGE}-token window", fatal=False)
        got = self.pool.alloc(need)
        if got is None:
            raise BackendError("KV page pool exhausted", fatal=False)
        base = len(self.pages[slot])
        self.pages[slot].extend(got)
        self._host_writable()
        self.h_bt[slot, base:base + need] = torch.tensor(got, dtype=torch.int32)
        self.bt_dirty = True
        self.bt_dirty_slots.add(slot)

    def _flush_moves(self) -> None:
        """Applies the row moves that `commit_path` queued (accepted tree nodes to their positions), in order, before anything reads the
        caches again; more than the staging array holds go in several launches."""
        while self.moves:
            part, self.moves = self.moves[:256], self.moves[256:]
            self._host_writable()
            self.h_moves[:len(part)] = torch.tensor(part, dtype=torch.int32)
            self.d_moves[:len(part)].copy_(self.h_moves[:len(part)], non_blocking=True)
            self._uploaded()
            self.h2d_bytes += len(part) * 12
            self.m.move_kv_rows(self.d_moves, len(part))
            self.tree_moves += len(part)

    def _sync_bt(self) -> None:
        self._flush_moves()
        if self.bt_dirty:
            self.d_bt.copy_(self.h_bt, non_blocking=True)
            self._uploaded()
            self.h2d_bytes += self.h_bt.numel() * 4
            self.bt_dirty = False
            self.bt_dirty_slots.clear()

    # ------------------------------------------------------------------ image prompts
    def supports_media(self) -> bool:
        """Image rows ride on this class's own prefill path of one rank; the multi-token-prediction block's lagged rows do not carry them."""
        return (type(self).prefill_slices is DenseGpuBackend.prefill_slices and type(self)._run_prefill is DenseGpuBackend._run_prefill
                and type(self)._announce_window is DenseGpuBackend._announce_window and not self.mtp_draft)

    def set_media(self, slot, media) -> None:
        if media is None:
            self.media[slot], self.rope_delta[slot] = None, 0
            return
        if not self.supports_media():
            raise BackendError("this backend takes no image inputs", fatal=False)
        emb = torch.as_tensor(media.embeds).to(device=self.m.device, dtype=self.m.embed.dtype)
        if emb.ndim != 2 or emb.shape[1] != self.cfg.d_model or emb.shape[0] != len(media.rows):
            raise BackendError(f"image rows of shape {tuple(emb.shape)} do not fit {len(media.rows)} placeholders of width {self.cfg.d_model}", fatal=False)
        if getattr(self.cfg, "mrope_sections", None) is not None and media.pos3 is None:
            raise BackendError("this model rotates by (T, H, W) positions: the image prompt must bring them", fatal=False)
        self.media[slot] = (np.asarray(media.rows, dtype=np.int64), emb, None if media.pos3 is None else np.asarray(media.pos3, dtype=np.int32))
        self.rope_delta[slot] = int(media.rope_delta) if media.pos3 is not None else 0
        self.h2d_bytes += emb.numel() * emb.element_size()

    def _prefill_media(self, items, M):
        """-> (embed_rows, pos3) of a prefill forward over `items`, or (None, None) when none of their slots holds image rows."""
        if not any(self.media[slot] is not None for slot, _, _, _ in items):
            return None, None
        dev = self.m.device
        need3 = getattr(self.cfg, "mrope_sections", None) is not None
        p3 = np.empty((M, 3), dtype=np.int32) if need3 else None
        idx, emb, q0 = [], [], 0
        for slot, start, toks, _ in items:
            n, md = len(toks), self.media[slot]
            if need3:
                if md is not None and md[2] is not None:
                    p3[q0:q0 + n] = md[2][start:start + n]
                else:
                    p3[q0:q0 + n] = np.arange(start, start + n, dtype=np.int32)[:, None]
            if md is not None:
                lo, hi = np.searchsorted(md[0], start), np.searchsorted(md[0], start + n)
                if hi > lo:
                    idx.append(q0 + (md[0][lo:hi] - start))
                    emb.append(md[1][lo:hi])
            q0 += n
        er = None
        if idx:
            ii = np.concatenate(idx)
            er = (torch.as_tensor(ii, device=dev), torch.cat(emb, 0))
            self.media_rows += len(ii)
            self.h2d_bytes += ii.nbytes
        t3 = None
        if need3:
            t3 = torch.as_tensor(p3, device=dev).contiguous()
            self.h2d_bytes += p3.nbytes
        return er, t3

    def _fill_rows(self, specs) -> int:
        """specs: list of (slot, first_position, tokens).  Fills the pinned staging rows; returns M.  Rows after an image prompt rotate at
        position + the slot's delta (rows of the prompt itself keep their index: their (T, H, W) positions travel apart)."""
        self._host_writable()
        h = self.h_rows.numpy()
        r = 0
        if any(self.rope_delta[slot] for slot, _, _ in specs):
            for slot, p0, toks in specs:
                n = len(toks)
                pos = np.arange(p0, p0 + n, dtype=np.int64)
                pg = np.asarray(self.pages[slot], dtype=np.int64)[pos // PAGE]
                md = self.media[slot]
                plen = len(md[2]) if (md is not None and md[2] is not None) else 0
                h[0, r:r + n] = toks
                h[1, r:r + n] = np.where(pos >= plen, pos + self.rope_delta[slot], pos)
                h[2, r:r + n] = pg * PAGE + pos % PAGE
                h[3, r:r + n] = slot
                h[4, r:r + n] = pos + 1
                r += n
            return r
        if all(len(t) == 1 for _, _, t in specs):
            # plain decode (one row per sequence): no per-sequence numpy calls, one bulk assignment per array
            n = len(specs)
            pages = self.pages
            h[0, :n] = [t[0] for _, _, t in specs]
            pos = [p0 for _, p0, _ in specs]
            h[1, :n] = pos
            h[2, :n] = [pages[slot][p0 // PAGE] * PAGE + p0 % PAGE for slot, p0, _ in specs]
            h[3, :n] = [slot for slot, _, _ in specs]
            h[4, :n] = [p + 1 for p in pos]
            return n
        for slot, p0, toks in specs:
            n = len(toks)
            pos = np.arange(p0, p0 + n, dtype=np.int64)
            pg = np.asarray(self.pages[slot], dtype=np.int64)[pos // PAGE]
            h[0, r:r + n] = toks
            h[1, r:r + n] = pos
            h[2, r:r + n] = pg * PAGE + pos % PAGE
            h[3, r:r + n] = slot
            h[4, r:r + n] = pos + 1
            r += n
        return r

    def _upload_rows(self, M: int) -> None:
        self.d_rows[:, :M].copy_(self.h_rows[:, :M], non_blocking=True)
        self._uploaded()
        self.h2d_bytes += 5 * M * 4

    # ------------------------------------------------------------------ prefill
    def prefill_slice(self, slot, start, tokens, candidates, last):
        return self.prefill_slices([(slot, start, tokens, last)], candidates)[0]

    def prefill_slices(self, items, candidates):
        m = self.m
        self._flush_moves()
        for slot, start, toks, _ in items:
            if start != self.len[slot]:
                raise BackendError(f"prefill at {start} but slot {slot} holds {self.len[slot]} tokens", fatal=False)
            self._ensure(slot, start + len(toks))
        M = self._fill_rows([(s, st, t) for s, st, t, _ in items])
        if M > m.max_rows:
            raise BackendError(f"prefill slice of {M} rows exceeds the {m.max_rows}-row scratch", fatal=False)
        n = len(items)
        hp = self.h_pf.numpy()
        q0 = 0
        last_rows = []
        for i, (slot, start, toks, last) in enumerate(items):
            hp[0, i], hp[1, i], hp[2, i], hp[3, i] = slot, q0, len(toks), start
            q0 += len(toks)
            if last:
                last_rows.append(q0 - 1)
        er, p3 = self._prefill_media(items, M)
        rows = self._run_prefill(M, n, max(len(t) for _, _, t, _ in items), last_rows, candidates, **({"embed_rows": er, "pos3": p3} if (er or p3 is not None) else {}))
        if self.mtp_draft:
            self._mtp_after_trunk([(s, st, t) for s, st, t, _ in items], keep_all=False)
        for slot, start, toks, _ in items:
            self.len[slot] = start + len(toks)
            self.pending[slot] = 0
        outs = [None] * n
        if last_rows:
            k = 0
            for i, (_, _, _, last) in enumerate(items):
                if last:
                    outs[i] = rows[k]
                    k += 1
        self._check()
        return outs

    def _run_prefill(self, M, n, max_qlen, last_rows, candidates, embed_rows=None, pos3=None):
        """Uploads the staged rows and runs one prefill forward; returns the candidate rows of `last_rows` (or None)."""
        m = self.m
        self._upload_rows(M)
        self._sync_bt()
        self.d_pf[:, :n].copy_(self.h_pf[:, :n], non_blocking=True)
        self._uploaded()
        self.h2d_bytes += 4 * n * 4
        d = self.d_rows
        pf = dict(seq_ids=self.d_pf[0], q_start=self.d_pf[1], q_len=self.d_pf[2], pos0=self.d_pf[3], nseq=n, max_qlen=max_qlen)
        lr = torch.tensor(last_rows, dtype=torch.long, device=m.device) if last_rows else None
        kw = {}
        if embed_rows is not None:
            kw["embed_rows"] = embed_rows
        if pos3 is not None:
            kw["pos3"] = pos3
        try:
            logits = m.forward_rows(d[0, :M], d[1, :M], d[2, :M], d[3, :M], d[4, :M], self.d_bt, prefill=pf, logit_rows=lr,
                                    want_logits=bool(last_rows), **kw)
        except RuntimeError as e:
            if type(e).__name__ != "CacheFull":
                raise
            raise BackendError(str(e), fatal=False)
        return self._read_candidates(logits, candidates) if last_rows else None

    # ------------------------------------------------------------------ decode / verify window
    def step(self, reqs, candidates):
        m = self.m
        self._flush_moves()          # (a multi-rank backend tells the other ranks: before this window is announced)
        specs = []
        for r in reqs:
            if r.first_position != self.len[r.slot]:
                raise BackendError(f"window at {r.first_position} but slot {r.slot} holds {self.len[r.slot]} tokens", fatal=False)
            self._ensure(r.slot, r.first_position + len(r.tokens))
            self.pending[r.slot] = len(r.tokens)
            specs.append((r.slot, r.first_position, r.tokens))
        M = self._fill_rows(specs)
        if M > self.max_rows:
            raise BackendError(f"window of {M} rows exceeds {self.max_rows}", fatal=False)
        self.m.window_seq_rows = max(len(r.tokens) for r in reqs)
        max_ctx = max(r.first_position + len(r.tokens) for r in reqs)
        bucket = min(m.max_ctx_alloc, (max_ctx + CTX_BUCKET - 1) // CTX_BUCKET * CTX_BUCKET)
        count = max(1, min(64, candidates))
        self._announce_window(M, count, bucket)
        self._upload_rows(M)
        self._sync_bt()
        self._run_window(M, count, bucket)
        if self.mtp_draft:
            self._mtp_after_trunk(specs, keep_all=True, bucket=bucket)
        rows = self._download(M, count)
        self._check()
        out, k = [], 0
        for r in reqs:
            out.append(rows[k:k + len(r.tokens)])
            k += len(r.tokens)
        return out

    # ------------------------------------------------------------------ tree windows
    def supports_trees(self) -> bool:
        """Tree windows run on one rank (the tree arrays are not announced to a group), without the multi-token-prediction block (its
        lagged rows follow chain positions) and on a model whose caches the row copies handle."""
        return (type(self)._announce_window is DenseGpuBackend._announce_window and type(self).step is DenseGpuBackend.step and not self.mtp_draft
                and self.m.supports_trees())

    def _drop_private(self, slot: int) -> None:
        if self.tree_priv[slot]:
            self.pool.release(self.tree_priv[slot])
            self.tree_priv[slot] = []

    def step_tree(self, reqs, candidates):
        """One verify window of draft trees (reference crates/engine/src/lib.rs:212-432 step_tree; crates/cuda/csrc/attention.cu:443).

        Row i of a request stands at position p0 + depth(i).  The nodes of the tree's first chain (row i at depth i, parent i - 1) use the
        sequence's own slots, as a chain window's drafts do.  Every other node gets private pages for the page(s) its path lies in: its own
        K / V rows are written there at its position, and in every layer the committed rows of that page and the node's ancestors are copied
        beside them, so that the node's view of the cache is what a serial run over its path would hold.  The attention kernel reads the
        chunks below the tree through the sequence's block table, shared by all of its rows, and the rest through each row's private table.
        Row outputs therefore equal, bit for bit, those of one-row steps along the row's path."""
        m = self.m
        if not self.supports_trees():
            raise BackendError("this backend runs no tree windows", fatal=False)
        self._flush_moves()
        VW, CH = self.VBT_W, self.VBT_W // 2 * PAGE             # private-table width (pages), keys per attention chunk
        self._host_writable()
        h = self.h_rows.numpy()
        hb, hv, hs = self.h_tree_base.numpy(), self.h_vbt.numpy(), self.h_spread.numpy()
        r0, ns, deepest = 0, 0, 0
        for r in reqs:
            n, p0, slot = len(r.tokens), r.first_position, r.slot
            if p0 != self.len[slot]:
                raise BackendError(f"tree window at {p0} but slot {slot} holds {self.len[slot]} tokens", fatal=False)
            if n > 64 or r.parents[0] != -1 or any(not 0 <= r.parents[i] < i for i in range(1, n)):
                raise BackendError("a tree window holds at most 64 rows per sequence, parents before children", fatal=False)
            if r0 + n > self.max_rows:
                raise BackendError(f"window of more than {self.max_rows} rows", fatal=False)
            self._drop_private(slot)
            depth, spine = [0] * n, [True] * n
            for i in range(1, n):
                depth[i] = depth[r.parents[i]] + 1
                spine[i] = r.parents[i] == i - 1 and spine[i - 1]
            self._ensure(slot, p0 + max(depth) + 1)
            self._host_writable()
            pages = self.pages[slot]
            first_pi = (p0 + 1) // PAGE                            # the page the tree's first draft position lies in
            c0 = (p0 + 1) // CH * (CH // PAGE)                     # page index that entry 0 of a private table stands for
            row_slot, priv = [0] * n, [None] * n
            for i in range(n):
                P = p0 + depth[i]
                if spine[i]:
                    row_slot[i] = pages[P // PAGE] * PAGE + P % PAGE
                    continue
                got = self.pool.alloc(P // PAGE - first_pi + 1)
                if got is None:
                    self._drop_private(slot)
                    raise BackendError("KV page pool exhausted (private pages of a tree window)", fatal=False)
                self.tree_priv[slot].extend(got)
                priv[i] = {first_pi + j: pg for j, pg in enumerate(got)}
                row_slot[i] = priv[i][P // PAGE] * PAGE + P % PAGE
            for i in range(n):
                k = r0 + i
                for j in range(VW):
                    pi = c0 + j
                    hv[k, j] = priv[i][pi] if (priv[i] is not None and pi in priv[i]) else (pages[pi] if pi < len(pages) else 0)
                if priv[i] is None:
                    continue
                # private pages: the committed rows (and the anchor) of the page the first draft position lies in, then the ancestors
                if (p0 + 1) % PAGE != 0:
                    if ns >= hs.shape[0]:
                        raise BackendError("tree window: too many row copies", fatal=False)
                    hs[ns] = (pages[first_pi] * PAGE, priv[i][first_pi] * PAGE, p0 % PAGE + 1)
                    ns += 1
                a = r.parents[i]
                while a > 0:
                    P = p0 + depth[a]
                    if ns >= hs.shape[0]:
                        raise BackendError("tree window: too many row copies", fatal=False)
                    hs[ns] = (row_slot[a], priv[i][P // PAGE] * PAGE + P % PAGE, 1)
                    ns += 1
                    a = r.parents[a]
            h[0, r0:r0 + n] = r.tokens
            h[1, r0:r0 + n] = p0 + np.asarray(depth, dtype=np.int64) + self.rope_delta[slot]
            h[2, r0:r0 + n] = row_slot
            h[3, r0:r0 + n] = slot
            h[4, r0:r0 + n] = p0 + np.asarray(depth, dtype=np.int64) + 1
            hb[r0:r0 + n] = p0
            self.pending[slot] = n
            self.tree_p0[slot], self.tree_parents[slot], self.tree_slots[slot] = p0, list(r.parents), row_slot
            deepest = max(deepest, p0 + max(depth) + 1)
            r0 += n
        M = r0
        nsb = 64
        while nsb < ns:
            nsb *= 2                                               # the copy launch's size is part of the graph key: few distinct sizes
        hs[ns:nsb] = 0                                             # (a run of 0 rows copies nothing)
        m.window_seq_rows = max(len(r.tokens) for r in reqs)
        bucket = min(m.max_ctx_alloc, (deepest + CTX_BUCKET - 1) // CTX_BUCKET * CTX_BUCKET)
        count = max(1, min(64, candidates))
        self._announce_tree_window(M, count, bucket, nsb)
        self._upload_rows(M)
        self.d_tree_base[:M].copy_(self.h_tree_base[:M], non_blocking=True)
        self.d_vbt[:M].copy_(self.h_vbt[:M], non_blocking=True)
        self.d_spread[:nsb].copy_(self.h_spread[:nsb], non_blocking=True)
        self._uploaded()
        self.h2d_bytes += M * 4 * (1 + VW) + nsb * 12
        self._sync_bt()
        self._tree_n = nsb
        try:
            self._run_window(M, count, bucket)
        finally:
            self._tree_n = 0
        self.tree_windows += 1
        self.tree_copies += ns
        rows = self._download(M, count)
        self._check()
        out, k = [], 0
        for r in reqs:
            out.append(rows[k:k + len(r.tokens)])
            k += len(r.tokens)
        return out

    def commit_path(self, slot, rows):
        """Keeps the anchor and the path `rows` of the slot's last tree window: the node at window row rows[d - 1] becomes position p0 + d
        (its K / V rows are copied to that position's slot in every layer before the next forward reads the caches)."""
        n, parents, p0, row_slot = self.pending[slot], self.tree_parents[slot], self.tree_p0[slot], self.tree_slots[slot]
        prev = 0
        for r in rows:
            if parents is None or not 0 < r < n or parents[r] != prev:
                raise BackendError(f"commit_path: row {r} does not follow row {prev} in slot {slot}'s last tree window", fatal=False)
            prev = r
        pg = self.pages[slot]
        for d, r in enumerate(rows, 1):
            P = p0 + d
            dst = pg[P // PAGE] * PAGE + P % PAGE
            if row_slot[r] != dst:
                self.moves.append((row_slot[r], dst, 1))
        # the private pages go back to the pool now: the queued copies run before the next forward (see _flush_moves), and whoever gets a
        # page writes it in kernels queued after them
        self._drop_private(slot)
        self.len[slot] += 1 + len(rows)
        self.pending[slot] = 0
        self.tree_parents[slot] = self.tree_slots[slot] = None

    # ------------------------------------------------------------------ multi-token-prediction block: lagged rows and drafts
    def _mtp_after_trunk(self, specs, keep_all: bool, bucket: int | None = None) -> None:
        """The trunk has just run `specs` = [(slot, first position, tokens)] (rows in that order; m.h holds their final residual rows).  Runs the
        block on the rows one position earlier - (hidden of p0 - 1 kept from the slot's last window, token p0), (hidden p0, token p0 + 1), ... -
        and keeps this call's rows for the next one (`keep_all`: every row of a window, since the accepted count is not known yet; a prefill
        slice keeps its last row).  Rows past the accepted prefix of a window hold speculative KV that the next call rewrites."""
        m, W = self.m, self.MTP_W
        NS = self.max_slots * W
        self._host_writable()
        h, hk = self.h_mtp.numpy(), self.h_keep.numpy()
        n_rows = n_keep = 0
        r0 = 0
        seq_rows = 1
        for slot, p0, toks in specs:
            n = len(toks)
            pg = self.pages[slot]
            have = self.mtp_p0[slot] >= 0 and self.mtp_p0[slot] <= p0 - 1 < self.mtp_p0[slot] + self.mtp_n[slot]
            first = p0 - 1 if (have and p0 > 0) else p0
            cnt = p0 + n - 1 - first                     # block rows at positions first .. p0 + n - 2
            if cnt > 0:
                pos = np.arange(first, first + cnt, dtype=np.int64)
                a = n_rows
                h[0, a:a + cnt] = toks[first + 1 - p0:]                                  # the token AFTER each position
                h[1, a:a + cnt] = pos
                h[2, a:a + cnt] = np.asarray(pg, dtype=np.int64)[pos // PAGE] * PAGE + pos % PAGE
                h[3, a:a + cnt] = slot
                h[4, a:a + cnt] = pos + 1
                src = NS + r0 + (pos - p0)                                                # this call's trunk rows ...
                if first < p0:
                    src[0] = slot * W + (p0 - 1 - self.mtp_p0[slot])                     # ... and the kept row before them
                h[5, a:a + cnt] = src
                n_rows += cnt
                seq_rows = max(seq_rows, cnt)
            if keep_all:
                kn = min(n, W)
                hk[0, n_keep:n_keep + kn] = r0 + np.arange(kn)
                hk[1, n_keep:n_keep + kn] = slot * W + np.arange(kn)
                n_keep += kn
                self.mtp_p0[slot], self.mtp_n[slot] = p0, kn
            else:
                hk[0, n_keep], hk[1, n_keep] = r0 + n - 1, slot * W
                n_keep += 1
                self.mtp_p0[slot], self.mtp_n[slot] = p0 + n - 1, 1
            r0 += n
        M = r0
        self.d_mtp[:, :max(1, n_rows)].copy_(self.h_mtp[:, :max(1, n_rows)], non_blocking=True)
        self.d_keep[:, :n_keep].copy_(self.h_keep[:, :n_keep], non_blocking=True)
        self._uploaded()
        self.h2d_bytes += 6 * n_rows * 4 + 2 * n_keep * 8
        self.mtp_src[NS:NS + M].copy_(m.h[:M])
        if n_rows:
            torch.index_select(self.mtp_src, 0, self.d_mtp[5, :n_rows].long(), out=self.mtp_in[:n_rows])
        # keep this call's rows only after the gather has read the previous ones
        self.mtp_src.index_copy_(0, self.d_keep[1, :n_keep], m.h.index_select(0, self.d_keep[0, :n_keep]))
        d = self.d_mtp
        ctx_cap = bucket or m.max_ctx_alloc
        saved_rows = m.window_seq_rows
        for c0 in range(0, n_rows, 256):
            c1 = min(n_rows, c0 + 256)
            m.window_seq_rows = min(seq_rows, c1 - c0)
            m.mtp_forward(d[0, c0:c1], self.mtp_in[c0:c1], d[1, c0:c1], d[2, c0:c1], d[3, c0:c1], d[4, c0:c1], self.d_bt, max_ctx=ctx_cap, want_logits=False)
        m.window_seq_rows = saved_rows
        self.mtp_rows += n_rows

    def _mtp_propose(self, asks):
        from .backend import DraftOffer
        m, W = self.m, self.MTP_W
        live = [a for a in asks if self.mtp_p0[a.slot] >= 0 and self.mtp_p0[a.slot] <= self.len[a.slot] - 1 < self.mtp_p0[a.slot] + self.mtp_n[a.slot]
                and a.max_drafts > 0]
        if not live:
            return {}
        n = len(live)
        k = min(self.DK, max(a.max_drafts for a in live))
        self._host_writable()
        h = self.h_draft.numpy()
        hk = self.h_keep.numpy()
        top = 0
        for i, a in enumerate(live):
            slot, p0 = a.slot, self.len[a.slot]
            if p0 != len(a.context) - 1:
                raise BackendError(f"draft for slot {slot} at {len(a.context) - 1} but the slot holds {p0} tokens", fatal=False)
            self._ensure(slot, p0 + k + 1)
            pg = self.pages[slot]
            for j in range(k):
                pos = p0 - 1 + j                  # the block's row: hidden of `pos`, token pos + 1 -> predicts token pos + 2
                h[j, 0, i] = a.context[-1] if j == 0 else 0
                h[j, 1, i], h[j, 2, i], h[j, 3, i], h[j, 4, i] = pos + self.rope_delta[slot], pg[pos // PAGE] * PAGE + pos % PAGE, slot, pos + 1
            hk[0, i] = slot * W + (p0 - 1 - self.mtp_p0[slot])
            top = max(top, p0 + k)
        bucket = min(m.max_ctx_alloc, (top + CTX_BUCKET - 1) // CTX_BUCKET * CTX_BUCKET)
        self.d_draft[:k, :, :n].copy_(self.h_draft[:k, :, :n], non_blocking=True)
        self.d_keep[0, :n].copy_(self.h_keep[0, :n], non_blocking=True)
        self._uploaded()
        self.h2d_bytes += k * 5 * n * 4 + n * 8
        self._sync_bt()
        saved_rows, m.window_seq_rows = m.window_seq_rows, 1
        d = self.d_draft
        torch.index_select(self.mtp_src, 0, self.d_keep[0, :n], out=self.mtp_chain[:n])
        for j in range(k):
            ids = d[0, 0, :n] if j == 0 else self.d_draft_ids[j - 1, :n]
            logits, hid = m.mtp_forward(ids, self.mtp_chain[:n], d[j, 1, :n], d[j, 2, :n], d[j, 3, :n], d[j, 4, :n], self.d_bt, max_ctx=bucket)
            if m.cfg.vocab_padded != m.cfg.vocab:
                logits[:, m.cfg.vocab:] = float("-inf")
            m.K.topk(logits, 1, m.topk_scratch, self.d_draft_ids[j, :n].view(n, 1), self.d_draft_vals[j, :n].view(n, 1))
            self.mtp_chain[:n].copy_(hid)
        m.window_seq_rows = saved_rows
        self.h_draft_ids[:k, :n].copy_(self.d_draft_ids[:k, :n], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes += k * n * 4
        self.draft_steps += k
        out = self.h_draft_ids.numpy()
        return {a.slot: DraftOffer([int(out[j, i]) for j in range(min(k, a.max_drafts))]) for i, a in enumerate(live)}

    # ------------------------------------------------------------------ window with device-side sampling and acceptance
    def supports_device_sampler(self) -> bool:
        return True

    def step_sampled(self, reqs, candidates, samplings):
        """Like `step`, but the keyed samples and the accepted-draft counts are computed on the device (verify kernel) and only token ids
        come back.  samplings: per request (Sampling, absolute position of the first sample).  Returns per request (samples, accepted);
        samples is None for a sequence whose rows held a NaN logit."""
        m = self.m
        specs = []
        for r in reqs:
            if r.first_position != self.len[r.slot]:
                raise BackendError(f"window at {r.first_position} but slot {r.slot} holds {self.len[r.slot]} tokens", fatal=False)
            self._ensure(r.slot, r.first_position + len(r.tokens))
            self.pending[r.slot] = len(r.tokens)
            specs.append((r.slot, r.first_position, r.tokens))
        M = self._fill_rows(specs)
        if M > self.max_rows:
            raise BackendError(f"window of {M} rows exceeds {self.max_rows}", fatal=False)
        self.m.window_seq_rows = max(len(r.tokens) for r in reqs)
        max_ctx = max(r.first_position + len(r.tokens) for r in reqs)
        bucket = min(m.max_ctx_alloc, (max_ctx + CTX_BUCKET - 1) // CTX_BUCKET * CTX_BUCKET)
        count = max(1, min(64, candidates))
        self._announce_window(M, count, bucket)
        self._upload_rows(M)
        self._sync_bt()
        self._run_window(M, count, bucket)
        if self.mtp_draft:
            self._mtp_after_trunk(specs, keep_all=True, bucket=bucket)
        windows = [(s, pos, r.tokens) for r, (s, pos) in zip(reqs, samplings)]
        samples, accepted, err = m.K.verify_accept(m._ids_view(M, count), m._vals_view(M, count), windows, device=m.device)
        hs, ha = samples.cpu().tolist(), accepted.cpu().tolist()      # the stream-ordered copies also fence the step
        self.h_status.copy_(m.status)
        self.d2h_bytes += M * 4 + len(reqs) * 4 + 16
        self._check()
        bad = int(err.item()) != 0
        out, k = [], 0
        for r, a in zip(reqs, ha):
            n = len(r.tokens)
            out.append((None if bad else hs[k:k + n], a))
            k += n
        return out

    def _graph_key(self, M: int, count: int, bucket: int) -> tuple:
        return (M, count, bucket, getattr(self.m, "window_seq_rows", 1), self._tree_n)

    def _run_window(self, M: int, count: int, bucket: int) -> None:
        if not self.use_graphs:
            try:
                self._window(M, count, bucket)
            except RuntimeError as e:
                if type(e).__name__ != "CacheFull":
                    raise
                # paged experts: this window touches more experts of one layer than the slab has slots; the batch fails, the server lives
                raise BackendError(str(e), fatal=False)
            return
        key = self._graph_key(M, count, bucket)
        g = self.graphs.get(key)
        if g is None:
            g = self._capture(M, count, bucket)
            self.graphs[key] = g
        g.replay()
        self.graph_replays += 1
        self.replayed_kernels += self.graph_kernels[key]

    def _announce_window(self, M: int, count: int, bucket: int) -> None:
        """Hook for multi-rank backends: tell the other ranks what is about to run (before the block-table dirty set is cleared)."""

    def _announce_tree_window(self, M: int, count: int, bucket: int, tree_n: int) -> None:
        """The same for a window of draft trees (the tree arrays are staged by then)."""

    def _window(self, M: int, count: int, bucket: int) -> None:
        d = self.d_rows
        tree = (self.d_tree_base[:M], self.d_vbt[:M], self.d_spread, self._tree_n) if self._tree_n else None
        logits = self.m.forward_rows(d[0, :M], d[1, :M], d[2, :M], d[3, :M], d[4, :M], self.d_bt, max_ctx=bucket, **({"tree": tree} if tree else {}))
        self.m.candidates(logits, count)

    def _capture(self, M: int, count: int, bucket: int):
        # one eager run first: sets function attributes, resolves driver entry points, warms the allocator
        self._window(M, count, bucket)
        torch.cuda.synchronize()
        from ..ops import lib as _oplib
        g = torch.cuda.CUDAGraph()
        n0 = _oplib.launch_count
        with torch.cuda.graph(g):
            self._window(M, count, bucket)
        self.graph_kernels[self._graph_key(M, count, bucket)] = _oplib.launch_count - n0
        self.graph_captures += 1
        return g

    def _download(self, M: int, count: int):
        ids, vals = self.m._ids_view(M, count), self.m._vals_view(M, count)
        hi, hv = self.h_cand_ids.view(-1)[:M * count].view(M, count), self.h_cand_vals.view(-1)[:M * count].view(M, count)
        hi.copy_(ids, non_blocking=True)
        hv.copy_(vals, non_blocking=True)
        self.h_status.copy_(self.m.status, non_blocking=True)   # bounded-wait status words ride along with the candidates
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes += M * count * 8 + 16
        a, b = hi.numpy().astype(np.uint32), hv.numpy().copy()
        return [RowOutput(a[i], b[i]) for i in range(M)]

    def _read_candidates(self, logits, candidates):
        count = max(1, min(64, candidates))
        R = logits.shape[0]
        self.m.candidates(logits, count)
        return self._download(R, count)

    def _check(self) -> None:
        from ..utils import canary
        if canary.enabled():
            try:
                canary.check_all()
            except canary.CanaryError as e:
                self._err = BackendError(f"guard band damaged: {e}", fatal=True)
        s = self.h_status.tolist()
        if s[0] != 0:
            self.m.status[:4].zero_()
            self.h_status[:4].zero_()
            from ..ops.kernels import ST_ABORTED, ST_PEER_TIMEOUT, STATUS_NAMES
            self._err = BackendError(f"device status code {s[0]} ({STATUS_NAMES.get(s[0], '?')}) at site {s[1]} (block {s[2]})", fatal=True,
                                     group_lost=s[0] in (ST_PEER_TIMEOUT, ST_ABORTED))

    def take_error(self):
        e, self._err = self._err, None
        return e

    def commit(self, slot, keep):
        keep = min(keep, self.pending[slot])
        self.len[slot] += keep
        self.pending[slot] = 0

    def release(self, slot):
        if self.pages[slot]:
            self.pool.release(self.pages[slot])
        self.pages[slot] = []
        self.len[slot] = 0
        self.pending[slot] = 0
        self._drop_private(slot)
        self.tree_parents[slot] = self.tree_slots[slot] = None
        self.media[slot], self.rope_delta[slot] = None, 0
        if self.mtp_draft:
            self.mtp_p0[slot], self.mtp_n[slot] = -1, 0
        self._host_writable()
        self.h_bt[slot].zero_()
        self.bt_dirty = True
        self.bt_dirty_slots.add(slot)

    # ------------------------------------------------------------------ prompt scoring
    def score_last(self, slot, tokens, chunk):
        """Prefill `tokens` into the empty slot in chunks; the last chunk returns the full logits row of the final position."""
        m = self.m
        if self.len[slot] != 0:
            raise BackendError(f"score on slot {slot}, which holds {self.len[slot]} tokens", fatal=False)
        chunk = min(chunk, m.max_rows)
        row = None
        for a in range(0, len(tokens), chunk):
            part = tokens[a:a + chunk]
            self._ensure(slot, a + len(part))
            M = self._fill_rows([(slot, a, part)])
            hp = self.h_pf.numpy()
            hp[0, 0], hp[1, 0], hp[2, 0], hp[3, 0] = slot, 0, M, a
            self._upload_rows(M)
            self._sync_bt()
            self.d_pf[:, :1].copy_(self.h_pf[:, :1], non_blocking=True)
            self._uploaded()
            d = self.d_rows
            pf = dict(seq_ids=self.d_pf[0], q_start=self.d_pf[1], q_len=self.d_pf[2], pos0=self.d_pf[3], nseq=1, max_qlen=M)
            last = a + len(part) >= len(tokens)
            lr = torch.tensor([M - 1], dtype=torch.long, device=m.device) if last else None
            logits = m.forward_rows(d[0, :M], d[1, :M], d[2, :M], d[3, :M], d[4, :M], self.d_bt, prefill=pf, logit_rows=lr, want_logits=last)
            self.len[slot] = a + len(part)
            if last:
                row = logits[0, :self.vocab_size].float().cpu().numpy()
        self.h_status.copy_(m.status)
        self._check()
        return row

    # ------------------------------------------------------------------ self-speculative drafter
    def supports_native_draft(self) -> bool:
        return self.self_draft or self.mtp_draft

    def _draft_chain(self, n: int, k: int, bucket: int) -> None:
        """k chained greedy draft steps over n sequences, ids handed from step to step on the device."""
        m, d = self.m, self.d_draft
        D = m.cfg.draft_layers
        for j in range(k):
            ids = d[0, 0, :n] if j == 0 else self.d_draft_ids[j - 1, :n]
            logits = m.forward_rows(ids, d[j, 1, :n], d[j, 2, :n], d[j, 3, :n], d[j, 4, :n], self.d_bt, max_ctx=bucket, n_layers=D)
            if m.cfg.vocab_padded != m.cfg.vocab:
                logits[:, m.cfg.vocab:] = float("-inf")
            # the level's LAT_K best candidates (value desc, id asc): the first feeds the next step, all of them form the offer's lattice
            m.K.topk(logits, self.LAT_K, m.topk_scratch, self.d_lat_ids[j, :n], self.d_lat_vals[j, :n])
            self.d_draft_ids[j, :n].copy_(self.d_lat_ids[j, :n, 0])

    def propose_batch(self, asks):
        if self.mtp_draft and asks:
            return self._mtp_propose(asks)
        if not self.self_draft or not asks:
            return {}
        from .backend import DraftOffer
        n = len(asks)
        k = min(self.DK, max(a.max_drafts for a in asks))
        if k <= 0:
            return {}
        self.m.window_seq_rows = 1          # draft steps feed one row per sequence
        self._host_writable()
        h = self.h_draft.numpy()
        top = 0
        for i, a in enumerate(asks):
            slot, p0 = a.slot, self.len[a.slot]
            if p0 != len(a.context) - 1:
                raise BackendError(f"draft for slot {slot} at {len(a.context) - 1} but the slot holds {p0} tokens", fatal=False)
            self._ensure(slot, p0 + k + 1)
            pg = self.pages[slot]
            for j in range(k):
                pos = p0 + j
                h[j, 0, i] = a.context[-1] if j == 0 else 0
                h[j, 1, i], h[j, 2, i], h[j, 3, i], h[j, 4, i] = pos + self.rope_delta[slot], pg[pos // PAGE] * PAGE + pos % PAGE, slot, pos + 1
            top = max(top, p0 + k)
        bucket = min(self.m.max_ctx_alloc, (top + CTX_BUCKET - 1) // CTX_BUCKET * CTX_BUCKET)
        self.d_draft[:k, :, :n].copy_(self.h_draft[:k, :, :n], non_blocking=True)
        self._uploaded()
        self.h2d_bytes += k * 5 * n * 4
        self._sync_bt()
        if self.use_graphs:
            key = (n, k, bucket)
            g = self.draft_graphs.get(key)
            if g is None:
                self._draft_chain(n, k, bucket)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._draft_chain(n, k, bucket)
                self.draft_graphs[key] = g
            g.replay()
        else:
            self._draft_chain(n, k, bucket)
        self.h_lat_ids[:k, :n].copy_(self.d_lat_ids[:k, :n], non_blocking=True)
        self.h_lat_vals[:k, :n].copy_(self.d_lat_vals[:k, :n], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes += k * n * self.LAT_K * 8
        self.draft_steps += k
        from ..spec.tree import Lattice
        ids, vals = self.h_lat_ids.numpy(), self.h_lat_vals.numpy()
        offers = {}
        for i, a in enumerate(asks):
            kk = min(k, a.max_drafts)
            offers[a.slot] = DraftOffer([int(ids[j, i, 0]) for j in range(kk)], [],
                                        Lattice([ids[j, i].tolist() for j in range(kk)], [vals[j, i].tolist() for j in range(kk)]),
                                        [float(vals[j, i, 0] - vals[j, i, 1]) for j in range(kk)])
        return offers

    # ------------------------------------------------------------------ prefix cache: pages are shared by refcount
    def prefix_block_tokens(self):
        return PAGE

    def prefix_bytes_per_block(self):
        return self.cfg.kv_bytes_per_token() * PAGE

    def prefix_commit(self, slot, blocks):
        ids = self.pages[slot][:blocks]
        self.pool.retain(ids)
        return [("page", p) for p in ids]

    def prefix_restore(self, slot, handles):
        assert self.len[slot] == 0 and not self.pages[slot]
        ids = [p for _, p in handles]
        self.pool.retain(ids)
        self.pages[slot] = list(ids)
        self._host_writable()
        self.h_bt[slot, :len(ids)] = torch.tensor(ids, dtype=torch.int32)
        self.bt_dirty = True
        self.bt_dirty_slots.add(slot)
        self.len[slot] = len(ids) * PAGE
        return self.len[slot]

    def prefix_release(self, handles):
        self.pool.release([p for _, p in handles])

    def prefix_export(self, handle):
        self._flush_moves()
        """One page of every layer's K and V cache as bytes ([2 * layers with a cache, n_kv, 64, head_dim] in the cache's own dtype)."""
        m = self.m
        if getattr(m, "k_cache", None) is None:
            return None
        p = handle[1]
        parts = [c[p] for c in m.k_cache if c is not None] + [c[p] for c in m.v_cache if c is not None]
        out = torch.stack(parts).contiguous().view(torch.uint8).cpu()
        self.d2h_bytes += out.numel()
        blob = out.numpy().tobytes()
        if getattr(m, "kv_i8", False) or getattr(m, "kv_q4", False):     # an int8 / q4 page is its bytes plus the scales of every layer
            sc = torch.stack([t[p] for t in m.k_tscale if t is not None] + [t[p] for t in m.v_tscale if t is not None]).contiguous().view(torch.uint8).cpu()
            self.d2h_bytes += sc.numel()
            blob += sc.numpy().tobytes()
        return blob

    def prefix_import(self, payload):
        m = self.m
        if getattr(m, "k_cache", None) is None:
            return None
        caches = [c for c in m.k_cache if c is not None] + [c for c in m.v_cache if c is not None]
        page_bytes = caches[0][0].numel() * caches[0].element_size()
        scaled = getattr(m, "kv_i8", False) or getattr(m, "kv_q4", False)
        scales = ([t for t in m.k_tscale if t is not None] + [t for t in m.v_tscale if t is not None]) if scaled else []
        scale_bytes = scales[0][0].numel() * scales[0].element_size() if scales else 0
        if len(payload) != page_bytes * len(caches) + scale_bytes * len(scales):
            return None                     # written by a different model or cache format
        got = self.pool.alloc(1)
        if got is None:
            return None
        raw = torch.frombuffer(bytearray(payload), dtype=torch.uint8).to(m.device, non_blocking=False)
        src = raw[:page_bytes * len(caches)].view(len(caches), page_bytes)
        for i, c in enumerate(caches):
            c[got[0]].view(torch.uint8).view(-1).copy_(src[i])
        if scales:
            ssrc = raw[page_bytes * len(caches):].view(len(scales), scale_bytes)
            for i, t in enumerate(scales):
                t[got[0]].view(torch.uint8).view(-1).copy_(ssrc[i])
        self.h2d_bytes += len(payload)
        return ("page", got[0])

    def quiesce(self):
        self._flush_moves()
        torch.cuda.synchronize()

    def stats(self):
        out = dict(graph_replays=self.graph_replays, graph_captures=self.graph_captures, replayed_kernels=self.replayed_kernels, h2d_bytes=self.h2d_bytes, d2h_bytes=self.d2h_bytes,
                   free_pages=self.pool.free_blocks())
        if self.mtp_draft:
            out.update(mtp_rows=self.mtp_rows, draft_steps=self.draft_steps)
        if self.media_rows:
            out.update(media_rows=self.media_rows)
        if getattr(self.m, "paged", None) is not None:
            out.update({"expert_" + k: v for k, v in self.m.paged.stats().items()})
        if self.tree_windows:
            out.update(tree_windows=self.tree_windows, tree_moves=self.tree_moves, tree_copies=self.tree_copies)
        return out


class _SkipFirstReplay:
    """A captured window whose first replay is skipped: the eager run that preceded the capture already did that step's work."""

    def __init__(self, graph):
        self.graph, self.first = graph, True

    def replay(self):
        if self.first:
            self.first = False
            return
        self.graph.replay()


def deepest_snapshot(handles) -> int:
    """Index of the last handle of a chain that carries a state snapshot (-1: none): a recurrent backend can restore up to there."""
    return max((i for i, h in enumerate(handles) if h[2] is not None), default=-1)


class HybridGpuBackend(DenseGpuBackend):
    """Backend over a hybrid (Mamba2 / delta-net + attention) executor.

    Rollback: a window that carries draft rows runs the recurrent layers in record mode (the pools are only read; every layer keeps the
    window's in_proj and post-conv rows), and `commit` queues (first row, rows kept) per sequence; before the next backend call that reads
    or writes the pools, ONE replay launch per recurrent layer walks the kept rows again and stores state and conv history (the reference's
    record / commit split, crates/cuda/csrc/gdn.cu:253-322).  The replay is the window's own arithmetic on the recorded inputs, so the
    pools equal what a serial decode leaves, bit for bit.  A window without drafts stores its state directly; such a window must not run
    twice for one step, so the eager run before its graph capture stands in for that graph's first replay.  `rollback=False` turns the
    record path off (no draft rows are planned, no record buffers are allocated).

    Prefix cache: off unless `state_snapshots=True`.  With it, a block's handle is (page, snapshot or None): the KV pages of the attention
    layers are shared by refcount as in the dense backend, and the handle of the block where a prefill slice ended also holds clones of the
    slot's conv and state pool rows (the engine cuts a slice at the prompt's last block boundary for backends with `prefix_needs_cuts`).  A
    restore goes as deep as the last handle with a snapshot.  A snapshot costs the model's whole per-stream state (hundreds of MiB for the
    large configs), which `prefix_bytes_per_block` charges to every block."""
    name = "cuda-hybrid"

    def __init__(self, model, max_slots=None, use_graphs: bool = True, state_snapshots: bool = False, rollback: bool = True,
                 verify_snapshots: bool = False):
        super().__init__(model, max_slots=max_slots, use_graphs=use_graphs, self_draft=False)
        self.state_snapshots = bool(state_snapshots)
        # digest every snapshot when it is taken and check the pools against it after a restore (one device-to-host read per restore)
        self.verify_snapshots = bool(verify_snapshots)
        self.rollback = bool(rollback)
        self._rec_rows = None        # slot -> first row of the last recorded window (None: the last window stored its state itself)
        self._rec_M = 0
        self._commits = []           # (first row, rows kept) of the sequences committed since that window
        self.commit_replays = 0
        if self.rollback:
            model.enable_record(self.max_rows)
            self.h_seg = torch.zeros(2, self.max_rows, dtype=torch.int32).pin_memory()
            self.d_seg = torch.zeros(2, self.max_rows, dtype=torch.int32, device=model.device)

    def supports_rollback(self) -> bool:
        return self.rollback

    def supports_device_sampler(self) -> bool:
        return False

    # ------------------------------------------------------------------ record / commit
    def _graph_key(self, M, count, bucket):
        return super()._graph_key(M, count, bucket) + (self.m.ssm_mode,)

    def _flush_commits(self) -> None:
        """Replay the kept rows of the last recorded window into the pools (one launch per recurrent layer)."""
        segs = [(r0, k) for r0, k in self._commits if k > 0]
        self._commits = []
        M, self._rec_rows = self._rec_M, None
        if not segs:
            return
        self._host_writable()
        h = self.h_seg.numpy()
        n = len(segs)
        h[0, :n] = [r0 for r0, _ in segs]
        h[1, :n] = [k for _, k in segs]
        self.d_seg[:, :n].copy_(self.h_seg[:, :n], non_blocking=True)
        self._uploaded()
        self.h2d_bytes += 8 * n
        d = self.d_rows
        self.m.commit_rows(M, d[3, :M], d[1, :M], self.d_seg[0], self.d_seg[1], n)
        self.commit_replays += 1

    def step(self, reqs, candidates):
        self._flush_commits()
        K = self.m.K
        record = self.rollback and any(len(r.tokens) > 1 for r in reqs)
        self.m.ssm_mode = K.SCAN_RECORD if record else K.SCAN_FINAL
        try:
            out = super().step(reqs, candidates)
        finally:
            self.m.ssm_mode = K.SCAN_FINAL
        if record:
            self._rec_rows, r0 = {}, 0
            for r in reqs:
                self._rec_rows[r.slot] = r0
                r0 += len(r.tokens)
            self._rec_M = r0
        return out

    def commit(self, slot, keep):
        keep = min(keep, self.pending[slot])
        if self._rec_rows is not None and slot in self._rec_rows:
            self._commits.append((self._rec_rows.pop(slot), keep))
        super().commit(slot, keep)

    def release(self, slot):
        if self._rec_rows is not None:
            self._rec_rows.pop(slot, None)        # rows of a window that is dropped with its sequence
        super().release(slot)

    def prefill_slices(self, items, candidates):
        self._flush_commits()
        return super().prefill_slices(items, candidates)

    def score_last(self, slot, tokens, chunk):
        self._flush_commits()
        return super().score_last(slot, tokens, chunk)

    def stats(self):
        st = super().stats()
        st["commit_replays"] = self.commit_replays
        return st

    def _capture(self, M, count, bucket):
        g = super()._capture(M, count, bucket)
        # a recorded window stores nothing, so running it twice is harmless; one that stores its state must not be replayed for the same step
        return g if self.m.ssm_mode == self.m.K.SCAN_RECORD else _SkipFirstReplay(g)

    def prefix_block_tokens(self):
        return PAGE if self.state_snapshots else 0

    def prefix_needs_cuts(self) -> bool:
        return self.state_snapshots

    def prefix_bytes_per_block(self):
        return self.cfg.kv_bytes_per_token() * PAGE + self.cfg.state_bytes_per_slot()

    def _snapshot(self, slot):
        self._flush_commits()
        m = self.m
        snap = {li: (m.conv_pool[li][slot].clone(), m.ssm_pool[li][slot].clone()) for li in m.ssm_pool}
        if self.verify_snapshots:
            snap["digest"] = m.K.state_digest([t for li in sorted(m.ssm_pool) for t in snap[li]])
        return snap

    def prefix_commit(self, slot, blocks):
        ids = self.pages[slot][:blocks]
        self.pool.retain(ids)
        snap = self._snapshot(slot) if self.len[slot] == blocks * PAGE else None
        return [("hpage", p, snap if i == len(ids) - 1 else None) for i, p in enumerate(ids)]

    def prefix_restore(self, slot, handles):
        assert self.len[slot] == 0 and not self.pages[slot]
        self._flush_commits()
        best = deepest_snapshot(handles)
        if best < 0:
            return 0
        ids = [h[1] for h in handles[:best + 1]]
        self.pool.retain(ids)
        self.pages[slot] = list(ids)
        self._host_writable()
        self.h_bt[slot, :len(ids)] = torch.tensor(ids, dtype=torch.int32)
        self.bt_dirty = True
        self.bt_dirty_slots.add(slot)
        m = self.m
        snap = handles[best][2]
        for li in m.ssm_pool:
            conv, state = snap[li]
            m.conv_pool[li][slot].copy_(conv)
            m.ssm_pool[li][slot].copy_(state)
        if "digest" in snap:
            got = m.K.state_digest([t[slot] for li in sorted(m.ssm_pool) for t in (m.conv_pool[li], m.ssm_pool[li])])
            if not torch.equal(got, snap["digest"]):
                raise BackendError(f"the state restored into slot {slot} does not have the digest recorded with its snapshot", fatal=True)
        self.len[slot] = len(ids) * PAGE
        return self.len[slot]

    def prefix_release(self, handles):
        self.pool.release([h[1] for h in handles])

    def prefix_export(self, handle):
        self._flush_moves()
        return None

    def prefix_import(self, payload):
        return None

