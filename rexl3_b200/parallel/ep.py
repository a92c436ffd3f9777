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


# ====================================================================================================== token all-to-all
TP_MAX = 8


class A2aDesc(ctypes.Structure):
    """Twin of the C struct A2aDesc (ops/csrc/moe.cu); `rx_moe_a2a_desc_size` guards the layout."""
    _fields_ = [("ranks", ctypes.c_int), ("rank", ctypes.c_int), ("cap", ctypes.c_int), ("d", ctypes.c_int), ("e_lo", ctypes.c_int * (TP_MAX + 1)),
                ("rx_rows", ctypes.c_void_p * TP_MAX), ("rx_meta", ctypes.c_void_p * TP_MAX), ("rx_count", ctypes.c_void_p * TP_MAX),
                ("rx_flag", ctypes.c_void_p * TP_MAX), ("ret", ctypes.c_void_p * TP_MAX), ("ret_flag", ctypes.c_void_p * TP_MAX),
                ("send_count", ctypes.c_void_p), ("local_count", ctypes.c_void_p), ("epoch", ctypes.c_void_p), ("use_index", ctypes.c_uint)]


@dataclass
class A2aLayout:
    """Arena of one rank for the token all-to-all: per parity set (consecutive layers alternate, so a rank that is one exchange ahead of a peer
    never overwrites what the peer still reads) the receive regions [ranks][cap] of rows, their (expert, source pair) words and counts, the
    return buffer [cap] of f32 rows, and the two flag arrays; cap = rows_cap * top_k = the most pairs one source rank can send."""
    ranks: int
    rows_cap: int
    d: int
    top_k: int

    def __post_init__(self):
        off = 0

        def take(n):
            nonlocal off
            o = off
            off = (off + n + 255) // 256 * 256
            return o
        R, self.cap = self.ranks, self.rows_cap * self.top_k
        self.epoch = take(4)
        self.send_count = take(4 * R)
        self.local_count = take(8)
        self.rx_flag = take(4 * 2 * R)
        self.ret_flag = take(4 * 2 * R)
        self.rx_count = take(4 * 2 * R)
        self.rx_meta = take(8 * 2 * R * self.cap)
        self.rx_rows = take(2 * 2 * R * self.cap * self.d)
        self.ret = take(4 * 2 * self.cap * self.d)
        self.total = off


class A2aComm:
    """What the MoE executor needs for the token all-to-all: the epoch bump of a forward and the descriptor of a layer's exchange."""

    def __init__(self, group, rank: int, n_experts: int):
        if ctypes.sizeof(A2aDesc) != _lib.load().rx_moe_a2a_desc_size():
            raise _lib.KernelError("all-to-all descriptor layout differs from the library's")
        self.g, self.rank, self.R, self.L = group, rank, group.ranks, group.layout
        L, R = self.L, self.R
        self.me = group.base(rank, rank)
        self._desc = []
        for parity in (0, 1):
            t = A2aDesc()
            t.ranks, t.rank, t.cap, t.d = R, rank, L.cap, L.d
            for r in range(R + 1):
                t.e_lo[r] = expert_range(n_experts, r, R)[0] if r < R else n_experts
            for r in range(R):
                b = group.base(rank, r)
                t.rx_rows[r] = b + L.rx_rows + 2 * parity * R * L.cap * L.d
                t.rx_meta[r] = b + L.rx_meta + 8 * parity * R * L.cap
                t.rx_count[r] = b + L.rx_count + 4 * parity * R
                t.rx_flag[r] = b + L.rx_flag + 4 * parity * R
                t.ret[r] = b + L.ret + 4 * parity * L.cap * L.d
                t.ret_flag[r] = b + L.ret_flag + 4 * parity * R
            t.send_count, t.local_count, t.epoch = self.me + L.send_count, self.me + L.local_count, self.me + L.epoch
            self._desc.append(t)

    def begin(self) -> None:
        _lib.check(_lib.load().rx_tp_bump_epoch(ctypes.c_void_p(self.me + self.L.epoch), _lib.stream_ptr()), "rx_tp_bump_epoch")
        _lib.count()

    def desc(self, li: int) -> A2aDesc:
        t = self._desc[li & 1]
        t.use_index = li + 1
        return t

    def rx_rows_ptr(self, li: int) -> int:
        return self.me + self.L.rx_rows + 2 * (li & 1) * self.R * self.L.cap * self.L.d


def make_a2a_loopback(cfg, ranks: int, rows_cap: int, device="cuda"):
    """R A2aComm objects over one process / one GPU (tests: the ranks are stepped phase by phase)."""
    g = LoopbackGroup(A2aLayout(ranks, rows_cap, cfg.d_model, cfg.top_k), device)
    return [A2aComm(g, r, cfg.n_experts) for r in range(ranks)]


def make_a2a_ipc(cfg, rank: int, ranks: int, rows_cap: int, device, ctrl_group) -> A2aComm:
    return A2aComm(IpcGroup(A2aLayout(ranks, rows_cap, cfg.d_model, cfg.top_k), rank, device, group=ctrl_group), rank, cfg.n_experts)
