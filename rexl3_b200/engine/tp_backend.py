"""Tensor-parallel backend: rank 0 runs the engine (scheduler, sampler, prefix cache) and leads; every other rank runs
`follow()`, a loop that receives each step's row arrays and repeats the same launches on its shard.  The ranks never
exchange tensors through the host: activations move GPU to GPU inside the fused kernels, the control plane is one small
CPU broadcast per step (lockstep SPMD, as in the reference's TpLeader / run_follower, crates/model/src/tp_runtime.rs:1-30,
:470-560).

Message (int32, broadcast from rank 0 over a CPU process group):
  [op, M, count, bucket, nseq, max_qlen, n_last, n_dirty, payload_len, 0...]  followed in the same buffer (or, when it
  does not fit, in a second broadcast of payload_len words) by: rows [5, M], prefill table [4, nseq], last rows [n_last],
  and for every dirty block-table row: slot, then the row.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

from ..models.dense_tp import DenseTPShard
from ..utils import trace
from .backend import BackendError, RowOutput
from .gpu_backend import DenseGpuBackend

OP_STOP, OP_WINDOW, OP_PREFILL, OP_MARK, OP_SYNC, OP_TREE, OP_MOVES = 0, 1, 2, 3, 4, 5, 6
# OP_TREE: a window of draft trees.  Payload: the rows, the dirty block-table rows, then tree_base [M], the private tables [M x W] and the
# row copies [n x 3]; head[9] = n, head[10] = W.  OP_MOVES: head[1] = n row copies [n x 3] to apply to every layer's caches (an accepted path).
HEAD = 16
SMALL = 8192       # words of the fixed first broadcast


class _TpExec:
    """What leader and followers share: staging buffers on the rank's GPU, the graph cache, the launch sequences."""

    def __init__(self, shard: DenseTPShard, max_slots: int, use_graphs: bool, ctrl_group):
        self.sh, self.ctrl, self.use_graphs = shard, ctrl_group, use_graphs
        dev = shard.device
        R = shard.max_rows
        self.max_slots = max_slots
        self.x_rows_h = torch.zeros(5, R, dtype=torch.int32).pin_memory()
        self.x_rows = torch.zeros(5, R, dtype=torch.int32, device=dev)
        self.x_bt_h = torch.zeros(max_slots, shard.max_blocks, dtype=torch.int32).pin_memory()
        self.x_bt = torch.zeros(max_slots, shard.max_blocks, dtype=torch.int32, device=dev)
        self.x_pf_h = torch.zeros(4, max_slots, dtype=torch.int32).pin_memory()
        self.x_pf = torch.zeros(4, max_slots, dtype=torch.int32, device=dev)
        self.msg = torch.zeros(SMALL, dtype=torch.int32)
        self.x_tree = None          # (tree_base, private tables, row copies) staging: (host pinned, device) pairs, made on first use
        self.x_moves = None
        self.tp_graphs = {}
        self.tp_graph_kernels = {}
        self.marks = []
        self._staged = torch.cuda.Event()       # recorded after the last upload from the pinned arrays; waited for before the next host write
        self._staged_pending = False

    # ---- launches
    def tree_staging(self):
        if self.x_tree is None:
            from ..ops import kernels as _K
            dev, R, W = self.sh.device, self.sh.max_rows, _K.attn_vbt_width()
            mk = lambda *shape: (torch.zeros(*shape, dtype=torch.int32).pin_memory(), torch.zeros(*shape, dtype=torch.int32, device=dev))  # noqa: E731
            self.x_tree = (mk(R), mk(R, W), mk(4096, 3))
            self.x_moves = mk(256, 3)
        return self.x_tree

    def run_window_eager(self, M, count, bucket, tree_n=0):
        d = self.x_rows
        out = None
        tree = None
        if tree_n:
            (_, tb), (_, vbt), (_, spread) = self.tree_staging()
            tree = (tb[:M], vbt[:M], spread, tree_n)
        for p in self.sh.phases(d[0, :M], d[1, :M], d[2, :M], d[3, :M], d[4, :M], self.x_bt, max_ctx=bucket, cand_count=count, tree=tree):
            out = p()
        return out

    def run_window(self, M, count, bucket, tree_n=0) -> int:
        """Runs one decode / verify window; returns the number of kernels launched (replayed)."""
        from ..ops import lib as _oplib
        if not self.use_graphs:
            n0 = _oplib.launch_count
            self.run_window_eager(M, count, bucket, tree_n)
            return _oplib.launch_count - n0
        key = (M, count, bucket, getattr(self.sh, "window_seq_rows", 1), tree_n)
        g = self.tp_graphs.get(key)
        if g is None:
            self.run_window_eager(M, count, bucket, tree_n)       # every rank runs this in the same step, so peers are there
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            n0 = _oplib.launch_count
            with torch.cuda.graph(g):
                self.run_window_eager(M, count, bucket, tree_n)
            self.tp_graph_kernels[key] = _oplib.launch_count - n0
            self.tp_graphs[key] = g
            dist.barrier(group=self.ctrl)                 # capture time differs per rank: start the replay together
        g.replay()
        return self.tp_graph_kernels[key]

    def run_prefill(self, M, nseq, max_qlen, last_rows, count):
        d = self.x_rows
        pf = dict(seq_ids=self.x_pf[0], q_start=self.x_pf[1], q_len=self.x_pf[2], pos0=self.x_pf[3], nseq=nseq, max_qlen=max_qlen)
        lr = torch.tensor(last_rows, dtype=torch.long, device=self.sh.device) if last_rows else None
        out = None
        for p in self.sh.phases(d[0, :M], d[1, :M], d[2, :M], d[3, :M], d[4, :M], self.x_bt, prefill=pf, logit_rows=lr,
                                want_logits=bool(last_rows), cand_count=count if last_rows else None):
            out = p()
        return out

    def mark(self):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.marks.append(ev)

    # ---- follower side
    def apply(self, head, payload: np.ndarray) -> bool:
        op, M, count, bucket, nseq, max_qlen, n_last, n_dirty = (int(x) for x in head[:8])
        if op == OP_STOP:
            return False
        if op == OP_MARK:
            self.mark()
            return True
        if op == OP_SYNC:
            torch.cuda.synchronize()
            dist.barrier(group=self.ctrl)
            return True
        k = 0
        if self._staged_pending:
            self._staged.synchronize()          # the previous message's copies may still be queued behind its kernels
            self._staged_pending = False
        if op == OP_MOVES:
            self.tree_staging()
            mh, md = self.x_moves
            mh.numpy()[:M] = payload[:3 * M].reshape(M, 3)
            md[:M].copy_(mh[:M], non_blocking=True)
            self._staged.record()
            self._staged_pending = True
            self.sh.move_kv_rows(md, M)
            return True
        self.x_rows_h.numpy()[:, :M] = payload[k:k + 5 * M].reshape(5, M)
        k += 5 * M
        if nseq:
            self.x_pf_h.numpy()[:, :nseq] = payload[k:k + 4 * nseq].reshape(4, nseq)
            k += 4 * nseq
        last_rows = payload[k:k + n_last].tolist()
        k += n_last
        nb = self.sh.max_blocks
        bt = self.x_bt_h.numpy()
        for _ in range(n_dirty):
            bt[int(payload[k])] = payload[k + 1:k + 1 + nb]
            k += 1 + nb
        tree_n = 0
        if op == OP_TREE:
            tree_n, W = int(head[9]), int(head[10])
            (tbh, tbd), (vh, vd), (sh_, sd) = self.tree_staging()
            if W != vh.shape[1]:
                raise BackendError(f"the leader's private tables are {W} pages wide, this rank's {vh.shape[1]}", fatal=True)
            tbh.numpy()[:M] = payload[k:k + M]
            k += M
            vh.numpy()[:M] = payload[k:k + M * W].reshape(M, W)
            k += M * W
            sh_.numpy()[:tree_n] = payload[k:k + 3 * tree_n].reshape(tree_n, 3)
            k += 3 * tree_n
            tbd[:M].copy_(tbh[:M], non_blocking=True)
            vd[:M].copy_(vh[:M], non_blocking=True)
            sd[:tree_n].copy_(sh_[:tree_n], non_blocking=True)
        self.x_rows[:, :M].copy_(self.x_rows_h[:, :M], non_blocking=True)
        if n_dirty:
            self.x_bt.copy_(self.x_bt_h, non_blocking=True)
        if op not in (OP_WINDOW, OP_TREE):
            self.x_pf[:, :nseq].copy_(self.x_pf_h[:, :nseq], non_blocking=True)
        self._staged.record()
        self._staged_pending = True
        if op in (OP_WINDOW, OP_TREE):
            self.sh.window_seq_rows = max(1, max_qlen)     # a window's message carries its longest run of rows per sequence in this field
            self.run_window(M, count, bucket, tree_n)
        else:
            self.run_prefill(M, nseq, max_qlen, last_rows, count)
        return True

    def recv(self):
        dist.broadcast(self.msg, src=0, group=self.ctrl)
        head = self.msg[:HEAD].numpy().copy()
        n = int(head[8])
        if HEAD + n <= SMALL:
            return head, self.msg[HEAD:HEAD + n].numpy().copy()
        big = torch.zeros(n, dtype=torch.int32)
        dist.broadcast(big, src=0, group=self.ctrl)
        return head, big.numpy()


def follow(shard: DenseTPShard, max_slots: int, ctrl_group, use_graphs: bool = True, leave_after: int = 0) -> _TpExec:
    """Body of every rank but 0: repeat the leader's launches until it says stop.  Returns the executor (its `marks` hold
    the timing events the leader asked for).  `leave_after` (failure tests): return after that many messages, between two steps and with
    this rank's stream drained, as a rank that goes away would."""
    ex = _TpExec(shard, max_slots, use_graphs, ctrl_group)
    seen = 0
    while True:
        if leave_after and seen >= leave_after:
            break
        trace.tp_event("F", shard.rank, "wait", seen)
        head, payload = ex.recv()
        seen += 1
        trace.tp_event("F", shard.rank, f"recv_op{int(head[0])}", int(head[1]))
        if not ex.apply(head, payload):
            break
        trace.tp_event("F", shard.rank, f"launched_op{int(head[0])}", int(head[1]))
        st = None
        if int(head[0]) == OP_SYNC:
            st = shard.status.tolist()
            if st[0] != 0:
                raise BackendError(f"rank {shard.rank}: device status code {st[0]} at site {st[1]} (block {st[2]}, aux {st[3]})", fatal=True)
    torch.cuda.synchronize()
    return ex


class DenseTpBackend(DenseGpuBackend):
    """Rank 0.  Same bookkeeping as the single-GPU backend; the forward is this rank's shard, announced to the followers first."""
    name = "cuda-tp"

    def __init__(self, shard: DenseTPShard, max_slots: int, ctrl_group, use_graphs: bool = True):
        if shard.rank != 0:
            raise ValueError("the engine runs on rank 0; other ranks call follow()")
        shard.max_seqs = max_slots
        super().__init__(shard, max_slots=max_slots, use_graphs=use_graphs)
        self.ex = _TpExec(shard, max_slots, use_graphs, ctrl_group)
        # the executor's staging buffers ARE the backend's (one upload path)
        self.ex.x_rows_h, self.ex.x_rows = self.h_rows, self.d_rows
        self.ex.x_bt_h, self.ex.x_bt = self.h_bt, self.d_bt
        self.ex.x_pf_h, self.ex.x_pf = self.h_pf, self.d_pf
        self.ex.x_tree = ((self.h_tree_base, self.d_tree_base), (self.h_vbt, self.d_vbt), (self.h_spread, self.d_spread))
        self.ex.x_moves = (self.h_moves, self.d_moves)
        self.ctrl_bytes = 0
        self.commands = 0

    # ---- control plane
    def _send(self, op, M=0, count=0, bucket=0, nseq=0, max_qlen=0, last_rows=(), tree_n=0, moves=None):
        parts = []
        if op == OP_MOVES:
            parts.append(np.asarray(moves, dtype=np.int32).reshape(-1))
        if op in (OP_WINDOW, OP_PREFILL, OP_TREE):
            parts.append(self.h_rows.numpy()[:, :M].reshape(-1))
            if nseq:
                parts.append(self.h_pf.numpy()[:, :nseq].reshape(-1))
            parts.append(np.asarray(last_rows, dtype=np.int32))
            dirty = sorted(self.bt_dirty_slots)
            bt = self.h_bt.numpy()
            for s in dirty:
                parts.append(np.asarray([s], dtype=np.int32))
                parts.append(bt[s])
            if op == OP_TREE:
                parts += [self.h_tree_base.numpy()[:M], self.h_vbt.numpy()[:M].reshape(-1), self.h_spread.numpy()[:tree_n].reshape(-1)]
        else:
            dirty = []
        payload = np.concatenate(parts).astype(np.int32, copy=False) if parts else np.zeros(0, dtype=np.int32)
        msg = self.ex.msg.numpy()
        msg[:HEAD] = 0
        msg[:9] = [op, M, count, bucket, nseq, max_qlen, len(last_rows), len(dirty), payload.size]
        msg[9], msg[10] = tree_n, self.VBT_W
        fits = HEAD + payload.size <= SMALL
        if fits:
            msg[HEAD:HEAD + payload.size] = payload
        trace.tp_event("L", 0, f"send_op{op}", M)
        dist.broadcast(self.ex.msg, src=0, group=self.ex.ctrl)
        if not fits:
            dist.broadcast(torch.from_numpy(np.ascontiguousarray(payload)), src=0, group=self.ex.ctrl)
        self.ctrl_bytes += 4 * (HEAD + payload.size)
        self.commands += 1

    def stats(self):
        st = super().stats()
        st.update(tp_ranks=dist.get_world_size(group=self.ex.ctrl), ctrl_bytes=self.ctrl_bytes, tp_commands=self.commands)
        return st

    def _announce_window(self, M, count, bucket):
        self._send(OP_WINDOW, M, count, bucket, 0, getattr(self.m, "window_seq_rows", 1))

    def _announce_tree_window(self, M, count, bucket, tree_n):
        self._send(OP_TREE, M, count, bucket, 0, getattr(self.m, "window_seq_rows", 1), tree_n=tree_n)

    def supports_trees(self) -> bool:
        return True

    def _flush_moves(self) -> None:
        """An accepted path's row copies go to every rank (each applies them to its own KV heads) before the next launch is announced."""
        while self.moves:
            part, self.moves = self.moves[:256], self.moves[256:]
            self._send(OP_MOVES, len(part), moves=part)
            self._host_writable()
            self.h_moves[:len(part)] = torch.tensor(part, dtype=torch.int32)
            self.d_moves[:len(part)].copy_(self.h_moves[:len(part)], non_blocking=True)
            self._uploaded()
            self.m.move_kv_rows(self.d_moves, len(part))
            self.tree_moves += len(part)

    def step(self, reqs, candidates):
        return super().step(reqs, candidates)

    def _window(self, M, count, bucket):
        self.ex.run_window_eager(M, count, bucket, self._tree_n)

    def _capture(self, M, count, bucket):
        g = super()._capture(M, count, bucket)
        dist.barrier(group=self.ex.ctrl)
        return g

    def _download(self, M, count):
        sh = self.m
        ids, vals = sh.cand_ids[:M * count].view(M, count), sh.cand_vals[:M * count].view(M, count)
        hi, hv = self.h_cand_ids.view(-1)[:M * count].view(M, count), self.h_cand_vals.view(-1)[:M * count].view(M, count)
        hi.copy_(ids, non_blocking=True)
        hv.copy_(vals, non_blocking=True)
        self.h_status.copy_(sh.status, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes += M * count * 8 + 16
        a, b = hi.numpy().astype(np.uint32), hv.numpy().copy()
        return [RowOutput(a[i], b[i]) for i in range(M)]

    def _run_prefill(self, M, n, max_qlen, last_rows, candidates):
        count = max(1, min(64, candidates))
        self._send(OP_PREFILL, M, count, 0, n, max_qlen, last_rows)
        self._upload_rows(M)
        self._sync_bt()
        self.d_pf[:, :n].copy_(self.h_pf[:, :n], non_blocking=True)
        self._uploaded()
        self.h2d_bytes += 4 * n * 4
        self.ex.run_prefill(M, n, max_qlen, last_rows, count)
        return self._download(len(last_rows), count) if last_rows else None

    # a block's cache is spread over the ranks' shards: no single-rank export (the spill tier stays empty under tensor parallelism)
    def prefix_export(self, handle):
        return None

    def prefix_import(self, payload):
        return None

    # ---- bench / lifecycle helpers
    def mark(self):
        self._send(OP_MARK)
        self.ex.mark()

    def sync_all(self):
        """Drains every rank's stream and checks every rank's status words (a follower raises on its own error)."""
        self._send(OP_SYNC)
        torch.cuda.synchronize()
        dist.barrier(group=self.ex.ctrl)
        self.h_status.copy_(self.m.status)
        self._check()

    def stop(self):
        self._send(OP_STOP)

    def quiesce(self):
        self.sync_all()
