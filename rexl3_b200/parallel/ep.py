"""Expert parallelism over NVLink peer memory: every rank owns a contiguous range of experts, activations are replicated (the
attention part runs on every rank), so the "dispatch" needs no transfer and the "combine" is a one-shot all-reduce fused into
the top-k weighted sum: the combine kernel writes each rank's weighted partial rows straight into slot `rank` of every
rank's buffer, and the residual/norm kernel adds the slots in rank order.  Same ownership model as the reference
(crates/cuda/src/moe_owned.rs:1-30: owned experts only, outputs summed, disjoint support); NVLink pushes and flags
replace its NCCL all-reduce.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

from ..ops import lib as _lib
from .symm import IpcGroup, LoopbackGroup


@dataclass
class EpLayout:
    ranks: int
    rows_cap: int
    d: int

    def __post_init__(self):
        off = 0

        def take(n):
            nonlocal off
            o = off
            off = (off + n + 255) // 256 * 256
            return o
        R = self.ranks
        self.epoch = take(4)
        self.count = take(4 * 16)
        self.ar_flag = take(4 * 2 * R)
        self.ar = take(8 * 2 * R * self.rows_cap * self.d)      # (value, ticket) pairs
        self.total = off


def expert_range(n_experts: int, rank: int, ranks: int):
    """Contiguous ownership; the first n_experts % ranks ranks hold one more."""
    base, extra = divmod(n_experts, ranks)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


class EpComm:
    """What the MoE executor needs from the group: an epoch bump per forward and the combine target of a layer."""

    def __init__(self, group, rank: int):
        from ..models.moe import CombineDst
        # the same descriptor is handed to the combine kernel and to the finish-and-broadcast kernel: both layouts must be this one
        L_ = _lib.load()
        if not (ctypes.sizeof(CombineDst) == L_.rx_moe_combine_desc_size() == L_.rx_tp_bcast_desc_size()):
            raise _lib.KernelError("combine / broadcast descriptor layouts differ from the library's")
        self.g, self.rank, self.R = group, rank, group.ranks
        self.L = group.layout
        self._dst = []
        me = group.base(rank, rank)
        for parity in (0, 1):
            t = CombineDst()
            t.ranks, t.rank, t.rows_cap = self.R, rank, self.L.rows_cap
            for r in range(self.R):
                b = group.base(rank, r)
                t.dst[r] = b + self.L.ar + 8 * parity * self.R * self.L.rows_cap * self.L.d
                t.dst_flag[r] = b + self.L.ar_flag + 4 * parity * self.R
            t.local_count = me + self.L.count + 4 * parity
            t.epoch = me + self.L.epoch
            self._dst.append(t)
        self.me = me

    def begin(self) -> None:
        _lib.check(_lib.load().rx_tp_bump_epoch(ctypes.c_void_p(self.me + self.L.epoch), _lib.stream_ptr()), "rx_tp_bump_epoch")
        _lib.count()

    def combine_target(self, li: int, M: int):
        if M > self.L.rows_cap:
            raise ValueError(f"{M} rows exceed the {self.L.rows_cap}-row all-reduce slots")
        parity = li & 1
        t = self._dst[parity]
        t.use_index = li + 1
        ar = self.me + self.L.ar + 8 * parity * self.R * self.L.rows_cap * self.L.d
        flags = self.me + self.L.ar_flag + 4 * parity * self.R
        return t, ar, flags, self.R, self.L.rows_cap, self.me + self.L.epoch, li + 1


    def target(self, use: int, M: int):
        """Slot set of the `use`-th collective of a forward (parity alternates with `use`)."""
        if M > self.L.rows_cap:
            raise ValueError(f"{M} rows exceed the {self.L.rows_cap}-row all-reduce slots")
        parity = use & 1
        t = self._dst[parity]
        t.use_index = use
        ar = self.me + self.L.ar + 8 * parity * self.R * self.L.rows_cap * self.L.d
        return t, ar, self.me + self.L.ar_flag + 4 * parity * self.R, self.R, self.L.rows_cap, self.me + self.L.epoch, use

    def local_slot(self):
        return None


def make_ipc(cfg, rank: int, ranks: int, rows_cap: int, device, ctrl_group) -> EpComm:
    return EpComm(IpcGroup(EpLayout(ranks, rows_cap, cfg.d_model), rank, device, group=ctrl_group), rank)


def make_loopback(cfg, ranks: int, rows_cap: int, device="cuda"):
    """R EpComm objects over one process / one GPU (tests: the ranks are stepped one after another)."""
    g = LoopbackGroup(EpLayout(ranks, rows_cap, cfg.d_model), device)
    return [EpComm(g, r) for r in range(ranks)]
