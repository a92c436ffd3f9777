"""Routed experts paged from a record file into a fixed device slab, under the MoE executor.

`write_records` lays every (layer, expert) of a host model into one file: a record holds the expert's six tensors (gate|up trellis, input
signs, output scales; down trellis, input signs, output scales), each part on a 256-byte boundary, the record padded to whole 4 KiB pages.
`StackSlab` is the device side of `sched.expert_cache`: instead of one byte range per slot it keeps six STACKED tensors
(`[slots, ...]`, the layout the grouped GEMM and its neighbours index by expert id) and a fill scatters a record's parts into row `slot` of
each.  `PagedExperts` ties both to an `ExpertCache`: per layer it turns the router's expert ids into slot ids (a hit, or a fill from the
file that evicts an unpinned slot), and the executor runs the routed FFN over slot ids with the slab as "the experts" - the kernels are the
resident path's kernels, so a paged forward returns the resident forward's bits.

Behaviour parity: reference crates/cuda/src/expert_cache.rs:1-40 (fixed slab, leases, bounded prefetch, miss-rate counters).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from ..sched import expert_cache as ec

PARTS = ("gu_trellis", "gu_suh", "gu_svh", "dn_trellis", "dn_suh", "dn_svh")


@dataclass
class Layout:
    path: str
    index: dict                 # (layer, expert) -> (offset, nbytes)
    parts: list                 # [(name, offset in record, nbytes, shape, numpy dtype name)] - the same for every expert
    expert_bytes: int
    n_layers: int
    n_experts: int
    codebook: str


def _parts_of(gu, dn):
    return [np.ascontiguousarray(gu.trellis), np.ascontiguousarray(gu.suh, dtype=np.float16), np.ascontiguousarray(gu.svh, dtype=np.float16),
            np.ascontiguousarray(dn.trellis), np.ascontiguousarray(dn.suh, dtype=np.float16), np.ascontiguousarray(dn.svh, dtype=np.float16)]


def write_records(weights, path: str, overwrite: bool = False, tag: str = "") -> Layout:
    """weights: models.dense.HostWeights of an MoE model (layers with experts_gu / experts_down).  Writes the record file unless one of the
    expected size and the same `tag` is there already (and `overwrite` is off); -> Layout.  The tag (the pack's fingerprint) sits in
    `path + ".tag"`: a record file left by another pack of the same shape is rewritten, not trusted."""
    n_exp = len(weights.layers[0].experts_gu)
    if any(len(lay.experts_gu) != n_exp for lay in weights.layers):
        raise ValueError("every layer must hold the same number of experts")
    return write_records_of(path, list(range(len(weights.layers))), n_exp, PARTS,
                            lambda li, e: _parts_of(weights.layers[li].experts_gu[e], weights.layers[li].experts_down[e]),
                            weights.layers[0].experts_gu[0].codebook, overwrite, tag)


MX_PARTS = ("gu_w", "gu_s", "dn_w", "dn_s")


def write_mx_records(weights, path: str, overwrite: bool = False, tag: str = "") -> Layout:
    """The MXFP4 experts of a latent-attention MoE model (models.mla.HostMla: routed layers hold ex_gu / ex_down = [(nibbles, scales)]): one
    record per (routed layer, expert) with the gate|up nibbles and scale bytes and the down nibbles and scale bytes."""
    routed = [li for li, lay in enumerate(weights.layers) if lay.router is not None]
    if not routed:
        raise ValueError("the model has no routed layers")
    n_exp = len(weights.layers[routed[0]].ex_gu)

    def parts(li, e):
        lay = weights.layers[li]
        return [np.ascontiguousarray(lay.ex_gu[e][0]).view(np.uint8), np.ascontiguousarray(lay.ex_gu[e][1]),
                np.ascontiguousarray(lay.ex_down[e][0]).view(np.uint8), np.ascontiguousarray(lay.ex_down[e][1])]
    return write_records_of(path, routed, n_exp, MX_PARTS, parts, "mxfp4", overwrite, tag)


def write_records_of(path: str, layers: list, n_exp: int, names, get_parts, codebook: str, overwrite: bool = False, tag: str = "") -> Layout:
    """The general form: `get_parts(layer, expert)` -> the expert's tensors (numpy, in the order of `names`), the same shapes for every expert
    of every layer in `layers`."""
    import os
    first = get_parts(layers[0], 0)
    parts, off = [], 0
    for name, a in zip(names, first):
        parts.append((name, off, a.nbytes, tuple(a.shape), a.dtype.name))
        off = (off + a.nbytes + ec.PART_ALIGN - 1) // ec.PART_ALIGN * ec.PART_ALIGN
    expert_bytes = parts[-1][1] + parts[-1][2]
    record = (expert_bytes + ec.PAGE - 1) // ec.PAGE * ec.PAGE
    index, pos = {}, 0
    same_tag = os.path.exists(path + ".tag") and open(path + ".tag").read() == tag if tag else not os.path.exists(path + ".tag")
    if not overwrite and same_tag and os.path.exists(path) and os.path.getsize(path) == record * n_exp * len(layers):
        for li in layers:
            for e in range(n_exp):
                index[(li, e)] = (pos, expert_bytes)
                pos += record
        return Layout(path, index, parts, expert_bytes, len(layers), n_exp, codebook)
    with open(path, "wb") as f:
        for li in layers:
            for e in range(n_exp):
                buf = bytearray(record)
                for (name, o, n, shape, dt), a in zip(parts, get_parts(li, e)):
                    if a.shape != shape or a.dtype.name != dt:
                        raise ValueError(f"expert ({li}, {e}) part {name} has shape {a.shape} {a.dtype.name}, the first expert has {shape} {dt}")
                    buf[o:o + n] = a.tobytes()
                f.write(buf)
                index[(li, e)] = (pos, expert_bytes)
                pos += record
    if tag:
        with open(path + ".tag", "w") as f:
            f.write(tag)
    elif os.path.exists(path + ".tag"):
        os.remove(path + ".tag")
    return Layout(path, index, parts, expert_bytes, len(layers), n_exp, codebook)


class StackSlab(ec.Slab):
    """Six stacked device tensors with one row per slot; pinned staging per fill thread; fills on a copy stream of their own."""

    def __init__(self, cfg: ec.Config, layout: Layout, device="cuda"):
        import torch
        self.cfg, self.layout, self.torch = cfg, layout, torch
        self.t = {}
        for name, off, n, shape, dt in layout.parts:
            self.t[name] = torch.empty((cfg.slots,) + tuple(shape), dtype=getattr(torch, dt), device=device)
        self._st = [torch.empty(cfg.record_bytes, dtype=torch.uint8).pin_memory() for _ in range(cfg.fill_threads + 1)]
        self.stream = torch.cuda.Stream(device=device)

    def staging(self, i: int):
        return self._st[i].numpy()

    def write(self, slot: int, i: int, nbytes: int) -> None:
        torch = self.torch
        with torch.cuda.stream(self.stream):
            for name, off, n, shape, dt in self.layout.parts:
                self.t[name][slot].copy_(self._st[i][off:off + n].view(getattr(torch, dt)).view(shape), non_blocking=True)
            done = torch.cuda.Event()
            done.record()
        done.synchronize()          # the staging buffer is free for this thread's next fill and the slot is complete for every stream

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.t.values())


class PagedExperts:
    """The executor's handle: the cache, the slab's stacks, and the per-layer translation of expert ids to slot ids."""

    def __init__(self, layout: Layout, budget_bytes: int, device="cuda", fill_threads: int = 4, direct: bool = False):
        self.layout = layout
        self.cfg = ec.Config(expert_bytes=layout.expert_bytes, budget_bytes=int(budget_bytes), n_layers=1, fill_threads=fill_threads)
        if self.cfg.slots < 1:
            raise ValueError(f"an expert budget of {budget_bytes} bytes holds no record of {self.cfg.record_bytes} bytes")
        self.slab = StackSlab(self.cfg, layout, device)
        self.source = ec.FileSource(layout.path, layout.index, direct=direct)
        self.cache = ec.ExpertCache(self.cfg, self.source, self.slab)
        self.held = []                       # leases of the layer whose kernels were queued last
        self.last = {}                       # layer -> experts its last call used (the next call's prefetch hint)
        self.calls = 0
        self.cold = self.asked = 0           # experts that were not resident when a layer asked for them / experts asked for

    @property
    def slots(self) -> int:
        return self.cfg.slots

    def release_held(self) -> None:
        """Call when every kernel queued so far has run (the caller has just synchronised with the stream)."""
        for l in self.held:
            l.release()
        self.held = []

    def resolve(self, layer: int, expert_ids: np.ndarray) -> np.ndarray:
        """expert_ids: the ids the router picked for this call of `layer` (any shape).  Makes every distinct one resident and pins it until
        `release_held`; -> int32 table [n_experts]: slot of each expert that is needed (0 elsewhere: never read)."""
        uniq = np.unique(expert_ids)
        if len(uniq) > self.slots:
            raise ec.CacheFull(f"layer {layer} needs {len(uniq)} experts at once, the slab holds {self.slots}: raise the expert budget or lower the rows per call")
        table = np.zeros(self.layout.n_experts, dtype=np.int32)
        keys = [(layer, int(e)) for e in uniq]
        cold = [k for k in keys if not self.cache.resident(k)]
        self.cold += len(cold)
        self.asked += len(keys)
        # residents first (their leases pin them against the fills below), then the misses: queued together so that the fill threads read
        # them side by side, then waited for one by one
        for k in keys:
            if k not in cold:
                lease = self.cache.get(k)
                self.held.append(lease)
                table[k[1]] = lease.slot
        self.cache.prefetch(cold)
        for k in cold:
            lease = self.cache.get(k)
            self.held.append(lease)
            table[k[1]] = lease.slot
        nxt = self.last.get(layer + 1)
        if nxt is not None and len(nxt) + len(uniq) <= self.slots:
            self.cache.prefetch([(layer + 1, int(e)) for e in nxt])
        self.last[layer] = uniq
        self.calls += 1
        return table

    def stats(self) -> dict:
        s = self.cache.stats()
        s.update(calls=self.calls, asked=self.asked, cold=self.cold, cold_rate=(self.cold / self.asked) if self.asked else 0.0)
        return s

    def close(self) -> None:
        self.release_held()
        self.cache.close()
        self.source.close()
