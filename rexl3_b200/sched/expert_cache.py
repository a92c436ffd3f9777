"""Expert-granular page cache: routed experts that do not fit in device memory stay in the pack on NVMe and are paged into a FIXED slab, one
slot per expert record, as the router asks for them (reference crates/cuda/src/expert_cache.rs:1-40).

Shape.  `ExpertCache` owns `budget_bytes // expert_bytes` slots (rounded down to a multiple of the layer count, so every layer can hold the
same number); nothing grows with demand.  `get(key)` returns a `Lease` on a resident slot - a hit, or a miss that evicts one unpinned slot
and fills it - and a lease pins its slot until it is released (a lease is what the grouped GEMM reads from).  `prefetch(keys)` queues misses
on a BOUNDED queue drained by fill threads, so a step can issue its fills and run attention / the shared expert while the reads land; a full
queue drops the hint (counted) instead of blocking.  Eviction is least-frequently-used with periodic ageing (counts halve every
`age_every` touches), because a decode trace re-touches a few hot experts per layer and LRU lets one prefill sweep flush them.  `stats()`
carries hits, misses, bytes read, evictions, dropped hints and the miss rate - the number that says whether serving from NVMe is viable.

Reads go through an `ExpertSource` and writes through a `Slab`, so the whole policy (eviction, pinning, queue, counters) runs on the host with
a fake file and a fake device; `DeviceSlab` is the only CUDA-dependent part: pinned staging buffers, one copy stream, `cudaMemcpyAsync` per
fill.  Allocation is accounted in one place: `Config.slab_bytes` (device) and `Config.staging_bytes` (pinned host); neither depends on the trace.
"""
from __future__ import annotations

import os
import queue
import threading
from dataclasses import dataclass

PAGE = 4096
PART_ALIGN = 256          # every part of an expert record starts on this boundary (what a device allocation guarantees)


class CacheFull(RuntimeError):
    """Every slot is pinned by a lease: the caller holds more experts at once than the slab has slots."""


@dataclass(frozen=True)
class Config:
    expert_bytes: int
    budget_bytes: int
    n_layers: int = 1
    queue_depth: int = 256
    fill_threads: int = 4
    age_every: int = 4096

    @property
    def record_bytes(self) -> int:
        return (self.expert_bytes + PAGE - 1) // PAGE * PAGE          # whole pages: O_DIRECT reads and aligned slots

    @property
    def slots(self) -> int:
        n = self.budget_bytes // self.record_bytes
        return n // max(1, self.n_layers) * max(1, self.n_layers)

    @property
    def slab_bytes(self) -> int:
        return self.slots * self.record_bytes

    @property
    def staging_bytes(self) -> int:
        return (self.fill_threads + 1) * self.record_bytes      # one per fill thread and one for the demand path


class ExpertSource:
    """Where expert records come from.  `read(key, buf)` fills `buf` (a writable buffer of record_bytes) and returns the bytes read."""

    def read(self, key, buf) -> int:
        raise NotImplementedError


class FileSource(ExpertSource):
    """Records inside one file: index {key: (offset, nbytes)}.  `direct=True` opens with O_DIRECT (offsets and sizes must then be page
    multiples and the buffer page-aligned, which DeviceSlab's pinned staging is)."""

    def __init__(self, path: str, index: dict, direct: bool = False):
        flags = os.O_RDONLY | (getattr(os, "O_DIRECT", 0) if direct else 0)
        self.fd = os.open(path, flags)
        self.index = dict(index)

    def read(self, key, buf) -> int:
        off, n = self.index[key]
        mv = memoryview(buf).cast("B")
        got = 0
        while got < n:
            r = os.preadv(self.fd, [mv[got:n]], off + got)
            if r <= 0:
                raise OSError(f"short read of expert {key!r}: {got} of {n} bytes")
            got += r
        return got

    def close(self) -> None:
        os.close(self.fd)


class Slab:
    """Where resident records live.  `staging(i)` is fill thread i's host buffer; `write(slot, i, nbytes)` moves it into the slot and returns
    when the slot may be read by work queued afterwards."""

    def staging(self, i: int):
        raise NotImplementedError

    def write(self, slot: int, i: int, nbytes: int) -> None:
        raise NotImplementedError


class HostSlab(Slab):
    """A slab in host memory (tests, and CPU backends)."""

    def __init__(self, cfg: Config):
        self.cfg = cfg
        self.mem = bytearray(cfg.slab_bytes)
        self._st = [bytearray(cfg.record_bytes) for _ in range(cfg.fill_threads + 1)]

    def staging(self, i: int):
        return self._st[i]

    def write(self, slot: int, i: int, nbytes: int) -> None:
        o = slot * self.cfg.record_bytes
        self.mem[o:o + nbytes] = self._st[i][:nbytes]

    def view(self, slot: int, nbytes: int) -> bytes:
        o = slot * self.cfg.record_bytes
        return bytes(self.mem[o:o + nbytes])


class DeviceSlab(Slab):
    """The slab in device memory: one uint8 tensor of slab_bytes, pinned staging per fill thread, fills on a copy stream of their own.
    `slot_ptr(slot)` is the device address a kernel reads the record from (256-byte aligned: records are whole pages)."""

    def __init__(self, cfg: Config, device="cuda"):
        import torch
        self.cfg, self.torch = cfg, torch
        self.mem = torch.empty(cfg.slab_bytes, dtype=torch.uint8, device=device)
        self._st = [torch.empty(cfg.record_bytes, dtype=torch.uint8).pin_memory() for _ in range(cfg.fill_threads + 1)]
        self.stream = torch.cuda.Stream(device=device)

    def staging(self, i: int):
        return self._st[i].numpy()

    def write(self, slot: int, i: int, nbytes: int) -> None:
        torch = self.torch
        o = slot * self.cfg.record_bytes
        with torch.cuda.stream(self.stream):
            self.mem[o:o + nbytes].copy_(self._st[i][:nbytes], non_blocking=True)
            done = torch.cuda.Event()
            done.record()
        done.synchronize()              # the staging buffer is reused by this thread's next fill; the slot is complete for every stream

    def slot_ptr(self, slot: int) -> int:
        return self.mem.data_ptr() + slot * self.cfg.record_bytes

    def view(self, slot: int, nbytes: int):
        o = slot * self.cfg.record_bytes
        return self.mem[o:o + nbytes]


class Lease:
    __slots__ = ("cache", "key", "slot", "_live")

    def __init__(self, cache, key, slot):
        self.cache, self.key, self.slot, self._live = cache, key, slot, True

    def release(self) -> None:
        if self._live:
            self._live = False
            self.cache._unpin(self.slot)

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.release()


class ExpertCache:
    def __init__(self, cfg: Config, source: ExpertSource, slab: Slab, sizes: "dict | None" = None):
        """sizes: {key: bytes of that record} (default: every record is expert_bytes)."""
        if cfg.slots < 1:
            raise ValueError(f"a budget of {cfg.budget_bytes} bytes holds no expert record of {cfg.record_bytes} bytes")
        self.cfg, self.source, self.slab, self.sizes = cfg, source, slab, sizes or {}
        self.lock = threading.Condition()
        self.slot_of: dict = {}                 # key -> slot (resident or being filled)
        self.key_of = [None] * cfg.slots
        self.pins = [0] * cfg.slots
        self.freq = [0] * cfg.slots
        self.filling: set = set()               # slots whose fill has not landed yet
        self.free = list(range(cfg.slots - 1, -1, -1))
        self.touches = 0
        self.hits = self.misses = self.bytes_read = self.evictions = self.hint_drops = self.hint_fills = 0
        self.q: "queue.Queue" = queue.Queue(maxsize=cfg.queue_depth)
        self._demand_lock = threading.Lock()
        self.threads = [threading.Thread(target=self._fill_loop, args=(i,), daemon=True, name=f"expert-fill-{i}") for i in range(cfg.fill_threads)]
        for t in self.threads:
            t.start()

    # ------------------------------------------------------------------ policy (lock held)
    def _touch(self, slot: int) -> None:
        self.freq[slot] += 1
        self.touches += 1
        if self.touches % self.cfg.age_every == 0:
            self.freq = [f >> 1 for f in self.freq]

    def _victim(self) -> int:
        if self.free:
            return self.free.pop()
        best = -1
        for s in range(self.cfg.slots):
            if self.pins[s] == 0 and s not in self.filling and (best < 0 or self.freq[s] < self.freq[best]):
                best = s
        if best < 0:
            raise CacheFull(f"all {self.cfg.slots} slots are pinned or being filled")
        del self.slot_of[self.key_of[best]]
        self.evictions += 1
        return best

    def _claim(self, key) -> int:
        """A slot for `key` that is about to be filled (pinned by the fill itself until it lands)."""
        slot = self._victim()
        self.slot_of[key], self.key_of[slot] = slot, key
        self.freq[slot] = 0
        self.filling.add(slot)
        return slot

    def _unpin(self, slot: int) -> None:
        with self.lock:
            self.pins[slot] -= 1
            self.lock.notify_all()

    # ------------------------------------------------------------------ fills
    def _fill(self, key, slot: int, i: int) -> None:
        n = int(self.sizes.get(key, self.cfg.expert_bytes))
        try:
            got = self.source.read(key, self.slab.staging(i))
            self.slab.write(slot, i, min(n, got))
        except BaseException:
            with self.lock:                  # the slot goes back unused; whoever waits for the key sees it gone and retries
                self.filling.discard(slot)
                if self.slot_of.get(key) == slot:
                    del self.slot_of[key]
                self.key_of[slot] = None
                self.free.append(slot)
                self.lock.notify_all()
            raise
        with self.lock:
            self.bytes_read += n
            self.filling.discard(slot)
            self.lock.notify_all()

    def _fill_loop(self, i: int) -> None:
        while True:
            item = self.q.get()
            if item is None:
                return
            key, slot = item
            try:
                self._fill(key, slot, i)
            except Exception:       # a failed hint is not fatal: the demand path reads the record again and raises there
                pass

    # ------------------------------------------------------------------ API
    def get(self, key) -> Lease:
        """Blocks until `key` is resident; the lease pins its slot."""
        with self.lock:
            while True:
                slot = self.slot_of.get(key)
                if slot is not None:
                    if slot in self.filling:
                        self.lock.wait(0.05)
                        continue
                    self.hits += 1
                    self._touch(slot)
                    self.pins[slot] += 1
                    return Lease(self, key, slot)
                self.misses += 1
                slot = self._claim(key)
                self.pins[slot] += 1
                self._touch(slot)
                break
        try:
            with self._demand_lock:           # one demand fill at a time shares the demand staging buffer
                self._fill(key, slot, self.cfg.fill_threads)
        except BaseException:
            with self.lock:
                self.pins[slot] -= 1
            raise
        return Lease(self, key, slot)

    def prefetch(self, keys) -> int:
        """Queues the misses among `keys`; returns how many were queued.  Never blocks: a full queue (or a slab with every slot pinned) drops
        the hint."""
        n = 0
        for key in keys:
            with self.lock:
                if key in self.slot_of:
                    continue
                try:
                    slot = self._claim(key)
                except CacheFull:
                    self.hint_drops += 1
                    continue
            try:
                self.q.put_nowait((key, slot))
                with self.lock:
                    self.hint_fills += 1
                n += 1
            except queue.Full:
                with self.lock:
                    self.hint_drops += 1
                    self.filling.discard(slot)
                    del self.slot_of[key]
                    self.key_of[slot] = None
                    self.free.append(slot)
        return n

    def resident(self, key) -> bool:
        with self.lock:
            s = self.slot_of.get(key)
            return s is not None and s not in self.filling

    def stats(self) -> dict:
        with self.lock:
            asks = self.hits + self.misses
            return dict(slots=self.cfg.slots, resident=len(self.slot_of), hits=self.hits, misses=self.misses, miss_rate=(self.misses / asks) if asks else 0.0,
                        bytes_read=self.bytes_read, evictions=self.evictions, hint_fills=self.hint_fills, hint_drops=self.hint_drops,
                        slab_bytes=self.cfg.slab_bytes, staging_bytes=self.cfg.staging_bytes)

    def close(self) -> None:
        for _ in self.threads:
            self.q.put(None)
        for t in self.threads:
            t.join(timeout=5)
