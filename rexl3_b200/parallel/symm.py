"""Symmetric peer memory for tensor parallelism: one arena per rank with the same layout everywhere, mapped into every
peer (CUDA IPC between processes, plain pointers between shards of one process), plus the descriptor structs the fused
kernels take.

Two groups implement the same interface:
  * ``IpcGroup``      - one process per GPU (torchrun); arenas exchanged as cudaIpcMemHandles over torch.distributed.
  * ``LoopbackGroup`` - R shards in ONE process on ONE GPU.  Kernels that wait on peers cannot run concurrently on one GPU,
    so the caller steps the shards phase by phase; every flag a kernel waits for has then already been written.  This is
    how the multi-rank protocol and numerics are tested without R GPUs (the reference's LoopbackComm plays the same role,
    crates/model/src/families/nemotron_h_omni/tp_comm.rs:433-830).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from ..ops import lib as _lib

TP_MAX = 8
c_u32p = ctypes.c_void_p


class GemmTp(ctypes.Structure):
    _fields_ = [("ranks", ctypes.c_int), ("rank", ctypes.c_int), ("strips_per_rank", ctypes.c_int), ("out_ld", ctypes.c_int),
                ("rows_cap", ctypes.c_int), ("out", ctypes.c_void_p * TP_MAX), ("out_flag", ctypes.c_void_p * TP_MAX),
                ("local_count", ctypes.c_void_p), ("in_flag", ctypes.c_void_p), ("in_cols_per_src", ctypes.c_int),
                ("epoch", ctypes.c_void_p), ("use_index", ctypes.c_uint)]


class FinishTp(ctypes.Structure):
    _fields_ = [("ranks", ctypes.c_int), ("rank", ctypes.c_int), ("in_flag", ctypes.c_void_p), ("ss", ctypes.c_void_p * TP_MAX),
                ("ss_flag", ctypes.c_void_p * TP_MAX), ("local_count", ctypes.c_void_p), ("epoch", ctypes.c_void_p),
                ("use_index", ctypes.c_uint), ("rows_cap", ctypes.c_int)]


class PushTp(ctypes.Structure):
    _fields_ = [("ranks", ctypes.c_int), ("rank", ctypes.c_int), ("ss", ctypes.c_void_p), ("ss_flag", ctypes.c_void_p),
                ("xr", ctypes.c_void_p * TP_MAX), ("xr_flag", ctypes.c_void_p * TP_MAX), ("local_count", ctypes.c_void_p),
                ("epoch", ctypes.c_void_p), ("use_index", ctypes.c_uint), ("rows_cap", ctypes.c_int)]


class CandTp(ctypes.Structure):
    _fields_ = [("ranks", ctypes.c_int), ("rank", ctypes.c_int), ("dst_ids", ctypes.c_void_p), ("dst_vals", ctypes.c_void_p),
                ("dst_flag", ctypes.c_void_p), ("epoch", ctypes.c_void_p), ("use_index", ctypes.c_uint), ("rows_cap", ctypes.c_int),
                ("id_offset", ctypes.c_int)]


class BcastTp(ctypes.Structure):
    _fields_ = [("ranks", ctypes.c_int), ("rank", ctypes.c_int), ("dst", ctypes.c_void_p * TP_MAX), ("dst_flag", ctypes.c_void_p * TP_MAX),
                ("local_count", ctypes.c_void_p), ("epoch", ctypes.c_void_p), ("use_index", ctypes.c_uint), ("rows_cap", ctypes.c_int)]


AR_ROWS = 256        # rows of a decode / verify window (the one-shot all-reduce path)
CAND_ROWS = 256      # rows of candidates one forward can return (the logits rows of a window)


def check_abi() -> None:
    L = _lib.load()
    a, b, c = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    L.rx_tp_desc_sizes(ctypes.byref(a), ctypes.byref(b), ctypes.byref(c))
    got = (ctypes.sizeof(GemmTp), ctypes.sizeof(FinishTp), ctypes.sizeof(PushTp))
    if got != (a.value, b.value, c.value):
        raise _lib.KernelError(f"TP descriptor layout mismatch: python {got}, library {(a.value, b.value, c.value)}")
    if ctypes.sizeof(CandTp) != L.rx_tp_cand_desc_size():
        raise _lib.KernelError("TP candidate descriptor layout mismatch")
    if ctypes.sizeof(BcastTp) != L.rx_tp_bcast_desc_size():
        raise _lib.KernelError("TP broadcast descriptor layout mismatch")


@dataclass
class ArenaLayout:
    """Byte offsets inside a rank's arena (identical on every rank)."""
    ranks: int
    rows_cap: int          # rows of the widest forward (prefill chunk)
    plane_elems: int       # max over row classes of splits * rows * n_own  (one source rank's planes of one site)
    d: int
    n_own: int

    def __post_init__(self):
        R = self.ranks
        off = 0

        def take(nbytes):
            nonlocal off
            o = off
            off = (off + nbytes + 255) // 256 * 256
            return o
        self.epoch = take(4)
        self.count = take(4 * 16)                      # local CTA counters: [0,1] part sites, [2,3] ss parities, [4,5] xr parities, [6,7] ar parities
        self.part_flag = take(4 * 2 * R)               # [site][src]
        self.ss_flag = take(4 * 2 * R)                 # [parity][src]
        self.xr_flag = take(4 * 2 * R)                 # [parity][src]
        self.ss = take(4 * 2 * R * self.rows_cap)      # [parity][src][row]
        self.part = take(4 * 2 * R * self.plane_elems)  # [site][src][plane]
        self.xr = take(2 * 2 * self.rows_cap * self.d)  # [parity][row][d] fp16
        self.ar_flag = take(4 * 2 * R)                 # [parity][src]
        self.ar = take(8 * 2 * R * AR_ROWS * self.d)   # [parity][src][row][d] (value, ticket) pairs: one-shot all-reduce slots
        self.cand_flag = take(4 * R)                   # [src]                      (read on the leader only)
        self.cand_ids = take(4 * R * CAND_ROWS * 64)   # [src][row * count + j] u32
        self.cand_vals = take(4 * R * CAND_ROWS * 64)
        self.total = off


class _GroupBase:
    ranks: int
    layout: ArenaLayout
    mm_local_base = 0      # this rank's address of the NVLink-multicast all-reduce buffer ([2 parities][AR_ROWS][d] f32), 0 = none
    mm_mc_base = 0         # the multicast address of the same buffer

    def mm_local(self, parity: int) -> int:
        return self.mm_local_base + 4 * parity * AR_ROWS * self.layout.d if self.mm_local_base else 0

    def mm_mc(self, parity: int) -> int:
        return self.mm_mc_base + 4 * parity * AR_ROWS * self.layout.d if self.mm_mc_base else 0

    def base(self, viewer: int, owner: int) -> int:
        """Device address of `owner`'s arena as seen from rank `viewer`."""
        raise NotImplementedError

    def local(self, rank: int) -> torch.Tensor:
        raise NotImplementedError

    # ---- descriptor builders (rank = the rank that will launch the kernel)
    def gemm_rs(self, rank: int, site: int, use_index: int, splits: int, rows: int) -> GemmTp:
        L, R = self.layout, self.ranks
        t = GemmTp()
        t.ranks, t.rank = R, rank
        t.strips_per_rank = L.n_own // 128
        t.out_ld, t.rows_cap = L.n_own, rows
        assert splits * rows * L.n_own <= L.plane_elems, "reduce-scatter planes exceed the arena"
        for r in range(R):
            b = self.base(rank, r)
            t.out[r] = b + L.part + 4 * site * R * L.plane_elems
            t.out_flag[r] = b + L.part_flag + 4 * site * R
        me = self.base(rank, rank)
        t.local_count = me + L.count + 4 * site
        t.in_flag, t.in_cols_per_src = None, 0
        t.epoch, t.use_index = me + L.epoch, use_index
        return t

    def gemm_ag(self, rank: int, parity: int, use_index: int, k: int) -> GemmTp:
        L, R = self.layout, self.ranks
        t = GemmTp()
        t.ranks, t.rank, t.strips_per_rank = R, rank, 0
        me = self.base(rank, rank)
        t.in_flag, t.in_cols_per_src = me + L.xr_flag + 4 * parity * R, k // R
        t.epoch, t.use_index = me + L.epoch, use_index
        return t

    def finish(self, rank: int, site: int, parity: int, use_index: int) -> FinishTp:
        L, R = self.layout, self.ranks
        t = FinishTp()
        t.ranks, t.rank, t.rows_cap = R, rank, L.rows_cap
        me = self.base(rank, rank)
        t.in_flag = me + L.part_flag + 4 * site * R
        for r in range(R):
            b = self.base(rank, r)
            t.ss[r] = b + L.ss + 4 * parity * R * L.rows_cap
            t.ss_flag[r] = b + L.ss_flag + 4 * parity * R
        t.local_count = me + L.count + 4 * (2 + parity)
        t.epoch, t.use_index = me + L.epoch, use_index
        return t

    def push(self, rank: int, parity: int, use_index: int) -> PushTp:
        L, R = self.layout, self.ranks
        t = PushTp()
        t.ranks, t.rank, t.rows_cap = R, rank, L.rows_cap
        me = self.base(rank, rank)
        t.ss = me + L.ss + 4 * parity * R * L.rows_cap
        t.ss_flag = me + L.ss_flag + 4 * parity * R
        for r in range(R):
            b = self.base(rank, r)
            t.xr[r] = b + L.xr + 2 * parity * L.rows_cap * L.d
            t.xr_flag[r] = b + L.xr_flag + 4 * parity * R
        t.local_count = me + L.count + 4 * (4 + parity)
        t.epoch, t.use_index = me + L.epoch, use_index
        return t

    def bcast(self, rank: int, parity: int, use_index: int) -> BcastTp:
        L, R = self.layout, self.ranks
        t = BcastTp()
        t.ranks, t.rank, t.rows_cap = R, rank, AR_ROWS
        for r in range(R):
            b = self.base(rank, r)
            t.dst[r] = b + L.ar + 8 * parity * R * AR_ROWS * L.d
            t.dst_flag[r] = b + L.ar_flag + 4 * parity * R
        me = self.base(rank, rank)
        t.local_count = me + L.count + 4 * (6 + parity)
        t.epoch, t.use_index = me + L.epoch, use_index
        return t

    def ar_ptr(self, rank: int, parity: int) -> int:
        return self.base(rank, rank) + self.layout.ar + 8 * parity * self.ranks * AR_ROWS * self.layout.d

    def ar_flag_ptr(self, rank: int, parity: int) -> int:
        return self.base(rank, rank) + self.layout.ar_flag + 4 * parity * self.ranks

    def cand(self, rank: int, leader: int, use_index: int, id_offset: int) -> CandTp:
        L = self.layout
        t = CandTp()
        t.ranks, t.rank, t.rows_cap, t.id_offset = self.ranks, rank, CAND_ROWS, id_offset
        b = self.base(rank, leader)
        t.dst_ids, t.dst_vals, t.dst_flag = b + L.cand_ids, b + L.cand_vals, b + L.cand_flag
        t.epoch, t.use_index = self.base(rank, rank) + L.epoch, use_index
        return t

    def part_ptr(self, rank: int, site: int) -> int:
        return self.base(rank, rank) + self.layout.part + 4 * site * self.ranks * self.layout.plane_elems

    def xr_view(self, rank: int, parity: int, rows: int) -> torch.Tensor:
        L = self.layout
        a = self.local(rank)
        off = L.xr + 2 * parity * L.rows_cap * L.d
        return a[off:off + 2 * rows * L.d].view(torch.float16).view(rows, L.d)

    def epoch_ptr(self, rank: int) -> int:
        return self.base(rank, rank) + self.layout.epoch


class LoopbackGroup(_GroupBase):
    def __init__(self, layout: ArenaLayout, device="cuda"):
        self.layout, self.ranks = layout, layout.ranks
        self.arenas = [torch.zeros(layout.total, dtype=torch.uint8, device=device) for _ in range(self.ranks)]

    def base(self, viewer, owner):
        return self.arenas[owner].data_ptr()

    def local(self, rank):
        return self.arenas[rank]


class _RawDeviceBuffer:
    """A cudaMalloc'ed range exposed to torch through the CUDA array interface (zero copy)."""

    def __init__(self, ptr: int, nbytes: int):
        self.ptr = ptr
        self.__cuda_array_interface__ = dict(shape=(nbytes,), typestr="|u1", data=(ptr, False), version=2)


class IpcGroup(_GroupBase):
    """One process per GPU.  Needs torch.distributed initialised (any backend) for the handle exchange.  The arena is its own
    cudaMalloc allocation (not a slice of torch's caching allocator), so the IPC handle maps exactly the arena."""

    def __init__(self, layout: ArenaLayout, rank: int, device, group=None):
        import torch.distributed as dist
        self.layout, self.ranks, self.rank = layout, layout.ranks, rank
        self._ctrl = group
        L = _lib.load()
        with torch.cuda.device(device):
            p = ctypes.c_void_p()
            _lib.check(L.rx_dev_alloc(layout.total, ctypes.byref(p)), "rx_dev_alloc")
            self._raw = _RawDeviceBuffer(p.value, layout.total)
            self.arena = torch.as_tensor(self._raw, device=device)
            assert self.arena.data_ptr() == p.value and self.arena.numel() == layout.total
            torch.cuda.synchronize()
        h = (ctypes.c_ubyte * 64)()
        _lib.check(L.rx_ipc_get_handle(ctypes.c_void_p(self.arena.data_ptr()), h), "rx_ipc_get_handle")
        handles = [None] * self.ranks
        dist.all_gather_object(handles, bytes(h), group=group)
        self.bases = []
        for r, hb in enumerate(handles):
            if r == rank:
                self.bases.append(self.arena.data_ptr())
                continue
            out = ctypes.c_void_p()
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(hb)
            _lib.check(L.rx_ipc_open(buf, ctypes.byref(out)), "rx_ipc_open")
            self.bases.append(out.value)
        dist.barrier(group=group)
        self._mm = None

    def enable_nvls(self) -> bool:
        """Binds a [2][AR_ROWS][d] f32 buffer to an NVLink multicast object (torch's symmetric-memory allocator does the driver work:
        cuMemCreate, handle exchange over the process group's store, cuMulticastCreate / BindMem) so that decode windows above the packet
        size can take their all-reduce from the switch (`multimem.ld_reduce`).  Collective: every rank calls it.  Returns False, and
        changes nothing, where the fabric has no multicast or NVLS is switched off (NCCL_NVLS_ENABLE=0 or RX_TP_NVLS=0: the setting of
        every failure test, since a rank that dies while bound to a multicast object can raise NVLink faults on its peers)."""
        import os
        import torch.distributed as dist
        if self.ranks < 2 or os.environ.get("NCCL_NVLS_ENABLE", "1") == "0" or os.environ.get("RX_TP_NVLS", "1") == "0":
            return False
        try:
            import torch.distributed._symmetric_memory as sm
            t = sm.empty(2 * AR_ROWS * self.layout.d, dtype=torch.float32, device=self.arena.device)
            hdl = sm.rendezvous(t, dist.group.WORLD)
            mc = int(hdl.multicast_ptr or 0)
        except Exception:        # no fabric support in this build / on this machine: keep the peer-store path
            return False
        ok = torch.tensor([1 if mc else 0], dtype=torch.int32)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self._ctrl)      # all ranks or none
        if int(ok[0]) == 0:
            return False
        t.zero_()
        torch.cuda.synchronize()
        self._mm, self.mm_local_base, self.mm_mc_base = (t, hdl), t.data_ptr(), mc
        return True

    def base(self, viewer, owner):
        assert viewer == self.rank
        return self.bases[owner]

    def local(self, rank):
        assert rank == self.rank
        return self.arena

    def close(self):
        L = _lib.load()
        for r, b in enumerate(self.bases):
            if r != self.rank:
                L.rx_ipc_close(ctypes.c_void_p(b))
        self.bases = []
        self.arena = None
        L.rx_dev_free(ctypes.c_void_p(self._raw.ptr))
