"""Expert page cache: policy, pinning, hints and counters on the host with a fake source; the device slab against a real file."""
import os
import threading

import pytest

from rexl3_b200.sched import expert_cache as ec


class FakeSource(ec.ExpertSource):
    def __init__(self, nbytes, fail=()):
        self.nbytes, self.reads, self.fail, self.gate = nbytes, [], set(fail), None

    def read(self, key, buf):
        if self.gate is not None:
            self.gate.wait(5)
        if key in self.fail:
            raise OSError(f"no record {key!r}")
        self.reads.append(key)
        mv = memoryview(buf).cast("B")
        layer, e = key
        mv[:self.nbytes] = bytes([(layer * 31 + e * 7 + i) % 251 for i in range(self.nbytes)])
        return self.nbytes


def _cache(slots=4, nbytes=100, **kw):
    cfg = ec.Config(expert_bytes=nbytes, budget_bytes=slots * ec.PAGE, n_layers=kw.pop("n_layers", 1), fill_threads=2, **kw)
    src = FakeSource(nbytes)
    slab = ec.HostSlab(cfg)
    return cfg, src, slab, ec.ExpertCache(cfg, src, slab)


def test_byte_accounting_and_slot_count():
    cfg = ec.Config(expert_bytes=7_720_000, budget_bytes=1 << 30, n_layers=40, fill_threads=4)
    assert cfg.record_bytes % ec.PAGE == 0 and cfg.record_bytes >= cfg.expert_bytes
    assert cfg.slots % 40 == 0 and cfg.slots * cfg.record_bytes <= 1 << 30 and cfg.slab_bytes == cfg.slots * cfg.record_bytes
    assert cfg.staging_bytes == 5 * cfg.record_bytes
    with pytest.raises(ValueError):
        ec.ExpertCache(ec.Config(expert_bytes=100, budget_bytes=10), FakeSource(100), None)


def test_hits_misses_bytes_and_lfu_eviction():
    cfg, src, slab, c = _cache(slots=3)
    try:
        for _ in range(5):                       # expert (0, 1) is hot
            c.get((0, 1)).release()
        c.get((0, 2)).release()
        c.get((0, 3)).release()
        with c.get((0, 4)) as lease:             # a fourth record: the coldest unpinned slot goes, not the hot one
            assert slab.view(lease.slot, 100) == bytes([(4 * 7 + i) % 251 for i in range(100)])
        assert c.resident((0, 1)) and not c.resident((0, 2))
        st = c.stats()
        assert (st["hits"], st["misses"], st["evictions"], st["bytes_read"]) == (4, 4, 1, 400) and st["miss_rate"] == 0.5
    finally:
        c.close()


def test_leases_pin_their_slots():
    cfg, src, slab, c = _cache(slots=2)
    try:
        a, b = c.get((0, 1)), c.get((0, 2))
        with pytest.raises(ec.CacheFull):
            c.get((0, 3))
        assert c.prefetch([(0, 3)]) == 0 and c.stats()["hint_drops"] == 1
        a.release()
        c.get((0, 3)).release()
        assert c.resident((0, 2)) and not c.resident((0, 1))
        b.release()
    finally:
        c.close()


def test_prefetch_fills_in_the_background_and_get_waits_for_a_fill_in_flight():
    cfg, src, slab, c = _cache(slots=4)
    try:
        src.gate = threading.Event()             # reads block until the gate opens
        assert c.prefetch([(0, 1), (0, 2), (0, 1)]) == 2
        assert not c.resident((0, 1))
        got = []
        t = threading.Thread(target=lambda: got.append(c.get((0, 1))))
        t.start()
        t.join(0.2)
        assert t.is_alive()                      # waiting for the fill, not reading the record a second time
        src.gate.set()
        t.join(5)
        assert got and c.resident((0, 2)) and sorted(src.reads) == [(0, 1), (0, 2)]
        got[0].release()
        st = c.stats()
        assert st["hits"] == 1 and st["misses"] == 0 and st["hint_fills"] == 2
    finally:
        src.gate.set()
        c.close()


def test_a_failed_read_frees_the_slot_and_raises_on_the_demand_path():
    cfg, src, slab, c = _cache(slots=2)
    try:
        src.fail.add((0, 9))
        with pytest.raises(OSError):
            c.get((0, 9))
        assert not c.resident((0, 9))
        c.get((0, 1)).release()
        c.get((0, 2)).release()                  # both slots are still usable
        assert c.stats()["resident"] == 2
    finally:
        c.close()


def test_ageing_halves_the_counts():
    cfg, src, slab, c = _cache(slots=2, age_every=8)
    try:
        for _ in range(7):
            c.get((0, 1)).release()
        c.get((0, 2)).release()                  # the 8th touch ages: 7 -> 3, 1 -> 0
        assert sorted(c.freq) == [0, 3]
    finally:
        c.close()


def test_file_source_reads_records(tmp_path):
    path = os.path.join(tmp_path, "bank.bin")
    rec = [bytes([k]) * ec.PAGE for k in range(3)]
    open(path, "wb").write(b"".join(rec))
    cfg = ec.Config(expert_bytes=ec.PAGE, budget_bytes=2 * ec.PAGE, fill_threads=1)
    src = ec.FileSource(path, {(0, k): (k * ec.PAGE, ec.PAGE) for k in range(3)})
    slab = ec.HostSlab(cfg)
    c = ec.ExpertCache(cfg, src, slab)
    try:
        for k in (2, 0, 1):
            with c.get((0, k)) as l:
                assert slab.view(l.slot, ec.PAGE) == rec[k]
    finally:
        c.close()
        src.close()


@pytest.mark.gpu
def test_device_slab_fills_from_a_file(tmp_path):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    path = os.path.join(tmp_path, "bank.bin")
    n = 3 * ec.PAGE + 512
    recs = [os.urandom(n) for _ in range(6)]
    stride = 4 * ec.PAGE
    with open(path, "wb") as f:
        for r in recs:
            f.write(r + b"\0" * (stride - n))
    cfg = ec.Config(expert_bytes=n, budget_bytes=4 * stride, n_layers=2, fill_threads=2)
    src = ec.FileSource(path, {(0, k): (k * stride, n) for k in range(6)})
    slab = ec.DeviceSlab(cfg)
    c = ec.ExpertCache(cfg, src, slab)
    try:
        c.prefetch([(0, 0), (0, 1)])
        for k in (0, 1, 2, 3, 4, 5, 0):
            with c.get((0, k)) as l:
                assert bytes(slab.view(l.slot, n).cpu().numpy().tobytes()) == recs[k]
                assert slab.slot_ptr(l.slot) % 256 == 0
        assert c.stats()["evictions"] >= 2
    finally:
        c.close()
        src.close()
