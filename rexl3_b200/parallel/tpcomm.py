"""One collective interface for code that is not fused with a GEMM: `TpComm` (reference crates/model/src/families/nemotron_h_omni/tp.rs:37-130).

    allreduce_sum_f32(buf)      in place, f32; every rank ends with the same bits (operands summed in rank order, except NcclTp: the library's order)
    allgather_f32(src, out)     out [ranks, n]
    swap_bytes(send, recv)      two ranks exchange a buffer
    barrier() / abort() / async_error() / capturable() / aux()

Implementations:
  SingleRank   one rank: every call is a no-op (all-gather copies).
  PeerTp       the product path on NVLink: symmetric arena (CUDA IPC across processes, or the loopback arena of one process), a rank pushes its
               buffer into its slot of every rank with plain peer stores and a ticket, every rank then sums / copies the slots it holds locally
               (ops/csrc/comm.cu `tp_coll_push_kernel`, `tp_coll_combine_kernel`).  One NVLink hop, bounded waits that report through the status
               words, capturable in a CUDA graph (tickets come from a device epoch).  Two slot sets alternate, so consecutive collectives need no
               barrier between them.
  NcclTp       torch.distributed (NCCL on GPUs, gloo on the CPU): the library baseline and the CPU test vehicle.
  loopback_group(n)  n PeerTp objects over one process / one GPU for tests.  Kernels that wait on one another must not run as separate launches
               on one GPU, so a loopback rank synchronises its stream and meets the others at a host barrier between the push and the combine:
               by the time a combine kernel runs, every ticket it looks for is already there.  Not capturable.
"""
from __future__ import annotations

import ctypes
import threading
from dataclasses import dataclass

import torch

from ..ops import lib as _lib

TP_MAX = 8


class CollTp(ctypes.Structure):
    """Twin of the C struct CollTp (ops/csrc/comm.cu); `rx_tp_coll_desc_size` guards the layout."""
    _fields_ = [("ranks", ctypes.c_int), ("rank", ctypes.c_int), ("cap", ctypes.c_longlong), ("slots", ctypes.c_void_p * TP_MAX), ("flags", ctypes.c_void_p * TP_MAX),
                ("local_count", ctypes.c_void_p), ("epoch", ctypes.c_void_p), ("use_index", ctypes.c_uint)]


class TpCommError(RuntimeError):
    pass


class TpComm:
    ranks: int = 1
    rank: int = 0

    def allreduce_sum_f32(self, buf: torch.Tensor) -> None:
        raise NotImplementedError

    def allgather_f32(self, src: torch.Tensor, out: torch.Tensor) -> None:
        raise NotImplementedError

    def swap_bytes(self, send: torch.Tensor, recv: torch.Tensor) -> None:
        raise NotImplementedError

    def barrier(self) -> None:
        pass

    def abort(self) -> None:
        pass

    def async_error(self) -> "str | None":
        return None

    def capturable(self) -> bool:
        return False

    def aux(self) -> "TpComm":
        """A second communicator for traffic that must not queue behind the main one (control-sized exchanges)."""
        return self


class SingleRank(TpComm):
    def allreduce_sum_f32(self, buf):
        pass

    def allgather_f32(self, src, out):
        out.view(-1)[:src.numel()].copy_(src.view(-1))

    def swap_bytes(self, send, recv):
        recv.copy_(send)

    def capturable(self):
        return True


class NcclTp(TpComm):
    """torch.distributed behind the interface (any initialised backend; `group` selects a process group)."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist, self.group = dist, group
        self.ranks, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self._err = None

    def allreduce_sum_f32(self, buf):
        assert buf.dtype == torch.float32
        self.dist.all_reduce(buf, op=self.dist.ReduceOp.SUM, group=self.group)

    def allgather_f32(self, src, out):
        if src.is_cuda:
            self.dist.all_gather_into_tensor(out.view(-1), src.contiguous().view(-1), group=self.group)
        else:
            self.dist.all_gather(list(out.view(self.ranks, -1).unbind(0)), src.contiguous().view(-1), group=self.group)

    def swap_bytes(self, send, recv):
        if self.ranks != 2:
            raise TpCommError("swap_bytes is a two-rank exchange")
        peer = 1 - self.rank
        ops = [self.dist.P2POp(self.dist.isend, send, peer, self.group), self.dist.P2POp(self.dist.irecv, recv, peer, self.group)]
        for r in self.dist.batch_isend_irecv(ops):
            r.wait()

    def barrier(self):
        self.dist.barrier(group=self.group)

    def capturable(self):
        return self.dist.get_backend(self.group) == "nccl"


@dataclass
class CollLayout:
    """Arena of one rank: epoch, CTA counter, two flag arrays and two slot sets [ranks][cap] of f32."""
    ranks: int
    cap: int                      # floats one collective may carry (a multiple of 4)

    def __post_init__(self):
        if self.cap < 4 or self.cap % 4:
            raise ValueError("the slot capacity is a positive multiple of 4 floats")
        off = 0

        def take(n):
            nonlocal off
            o = off
            off = (off + n + 255) // 256 * 256
            return o
        self.epoch, self.local_count = take(4), take(4)
        self.flags = take(4 * 2 * self.ranks)
        self.slots = take(4 * 2 * self.ranks * self.cap)
        self.total = off
        self.d = 0               # (symm._GroupBase reads it for the multicast buffer, which this layout does not use)


class PeerTp(TpComm):
    def __init__(self, group, rank: int, status: "torch.Tensor | None" = None, host_barrier: "threading.Barrier | None" = None, ctrl=None):
        """group: parallel.symm LoopbackGroup / IpcGroup over a CollLayout.  host_barrier: loopback ranks (threads of one process) meet there.
        ctrl: a torch.distributed group for `barrier()` between processes."""
        from ..ops import kernels as K
        L = _lib.load()
        if ctypes.sizeof(CollTp) != L.rx_tp_coll_desc_size():
            raise _lib.KernelError("collective descriptor layout differs from the library's")
        self.g, self.rank, self.ranks, self.L = group, rank, group.ranks, group.layout
        self.me = group.base(rank, rank)
        self.status = status if status is not None else K.new_status(group.local(rank).device)
        self.K = K
        self.host_barrier, self.ctrl = host_barrier, ctrl
        self.use = 0
        self._aborted = False
        self._desc = []
        lay = self.L
        for parity in (0, 1):
            t = CollTp()
            t.ranks, t.rank, t.cap = self.ranks, rank, lay.cap
            for r in range(self.ranks):
                b = group.base(rank, r)
                t.slots[r] = b + lay.slots + 4 * parity * self.ranks * lay.cap
                t.flags[r] = b + lay.flags + 4 * parity * self.ranks
            t.local_count, t.epoch = self.me + lay.local_count, self.me + lay.epoch
            self._desc.append(t)

    def _next(self) -> CollTp:
        """Collectives are numbered in launch order; 4095 of them share one epoch, then the epoch moves (every rank makes the same calls)."""
        if self.use % 4095 == 0:
            _lib.check(_lib.load().rx_tp_bump_epoch(ctypes.c_void_p(self.me + self.L.epoch), _lib.stream_ptr()), "rx_tp_bump_epoch")
        self.use += 1
        t = self._desc[self.use & 1]
        t.use_index = (self.use - 1) % 4095 + 1
        return t

    def _meet(self) -> None:
        if self.host_barrier is not None:        # loopback: every rank's push has completed before any combine kernel is launched
            torch.cuda.current_stream().synchronize()
            self.host_barrier.wait()

    def _run(self, src, dst, count, mode) -> None:
        if self._aborted:
            raise TpCommError("the communicator was aborted")
        if src.dtype != torch.float32 or not src.is_contiguous() or count % 4 or count > self.L.cap:
            raise TpCommError(f"collective of {count} floats: f32, contiguous, a multiple of 4 and at most {self.L.cap}")
        L, t = _lib.load(), self._next()
        _lib.check(L.rx_tp_coll_push(src.data_ptr(), count, ctypes.byref(t), _lib.stream_ptr()), "rx_tp_coll_push")
        self._meet()
        _lib.check(L.rx_tp_coll_combine(dst.data_ptr(), count, mode, self.status.data_ptr(), ctypes.byref(t), _lib.stream_ptr()), "rx_tp_coll_combine")
        _lib.count(2)
        if self.host_barrier is not None:        # a slot set is reused two collectives later: keep the loopback ranks within one of each other
            torch.cuda.current_stream().synchronize()
            self.host_barrier.wait()

    def allreduce_sum_f32(self, buf):
        self._run(buf, buf, buf.numel(), 0)

    def allgather_f32(self, src, out):
        if out.numel() != self.ranks * src.numel() or out.dtype != torch.float32 or not out.is_contiguous():
            raise TpCommError("all-gather output: f32 contiguous [ranks, n]")
        self._run(src, out, src.numel(), 1)

    def swap_bytes(self, send, recv):
        if self.ranks != 2:
            raise TpCommError("swap_bytes is a two-rank exchange")
        n = send.numel() * send.element_size()
        if n % 16 or n != recv.numel() * recv.element_size() or n // 4 > self.L.cap:
            raise TpCommError("swap_bytes: equal sizes, a multiple of 16 bytes, within the slot capacity")
        both = torch.empty(2, n // 4, dtype=torch.float32, device=send.device)
        self._run(send.contiguous().view(torch.uint8).view(torch.float32).view(-1), both, n // 4, 1)
        recv.view(torch.uint8).view(-1).copy_(both[1 - self.rank].view(torch.uint8).view(-1))

    def barrier(self):
        if self.host_barrier is not None:
            torch.cuda.current_stream().synchronize()
            self.host_barrier.wait()
        elif self.ctrl is not None:
            import torch.distributed as dist
            torch.cuda.current_stream().synchronize()
            dist.barrier(group=self.ctrl)

    def abort(self):
        """Raises the abort word: every bounded wait of this rank returns at once with status `aborted`."""
        self._aborted = True
        self.K.set_abort(self.status, True)

    def async_error(self):
        s = self.status.tolist()
        if s[0] == 0:
            return None
        return f"{self.K.STATUS_NAMES.get(s[0], s[0])} at site {s[1]}"

    def capturable(self):
        return self.host_barrier is None


def loopback_group(ranks: int, cap_floats: int, device="cuda") -> list:
    """`ranks` PeerTp objects over one process / one GPU; drive each from its own thread (the host barrier makes them meet)."""
    from .symm import LoopbackGroup
    g = LoopbackGroup(CollLayout(ranks, cap_floats), device)
    bar = threading.Barrier(ranks)
    return [PeerTp(g, r, host_barrier=bar) for r in range(ranks)]


def peer_group(rank: int, ranks: int, cap_floats: int, device, ctrl_group) -> PeerTp:
    """One process per GPU: the arena is mapped into every peer by CUDA IPC (handles travel over `ctrl_group`)."""
    from .symm import IpcGroup
    return PeerTp(IpcGroup(CollLayout(ranks, cap_floats), rank, device, group=ctrl_group), rank, ctrl=ctrl_group)
