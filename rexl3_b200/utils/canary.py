"""Guard bands around scratch and output buffers: with `REXL3_CANARY=1` every buffer allocated through `guarded()` sits between two bands of a
fixed byte pattern inside one allocation, and `check_all()` (one small device-to-host read per buffer) names the buffer and the side whose band
changed.  A kernel that writes past its buffer then shows up as a named error on the host instead of as silent corruption of a neighbour - the
stand-in for a memory checker on a pool where none may run (the write lands inside the same allocation, so nothing faults).  Off by default:
`guarded()` is then a plain allocation and `check_all()` does nothing."""
from __future__ import annotations

import os

import torch

BAND_BYTES = 4096
PATTERN = 0xA5


class CanaryError(RuntimeError):
    pass


_registry: list = []          # (name, whole uint8 tensor, payload bytes)


def enabled() -> bool:
    return os.environ.get("REXL3_CANARY", "0") == "1"


def guarded(name: str, shape, dtype, device, zero: bool = False, force: bool = False) -> torch.Tensor:
    """An uninitialised (or zeroed) tensor of `shape`; with canaries on, a view between two guard bands.  The view starts 4096 bytes into the
    allocation, so every alignment the plain allocation gave (256 bytes and more) is kept."""
    shape = tuple(shape) if isinstance(shape, (tuple, list, torch.Size)) else (int(shape),)
    if not (enabled() or force):
        return (torch.zeros if zero else torch.empty)(shape, dtype=dtype, device=device)
    n = 1
    for s in shape:
        n *= int(s)
    nbytes = n * torch.empty((), dtype=dtype).element_size()
    pad = (-nbytes) % 16
    whole = torch.empty(BAND_BYTES + nbytes + pad + BAND_BYTES, dtype=torch.uint8, device=device)
    whole[:BAND_BYTES].fill_(PATTERN)
    whole[BAND_BYTES + nbytes:].fill_(PATTERN)
    if zero:
        whole[BAND_BYTES:BAND_BYTES + nbytes].zero_()
    _registry.append((name, whole, nbytes))
    return whole[BAND_BYTES:BAND_BYTES + nbytes].view(dtype).view(shape)


def check_all() -> int:
    """Raises CanaryError naming every damaged band; returns the number of buffers checked."""
    bad = []
    for name, whole, nbytes in _registry:
        lo = whole[:BAND_BYTES]
        hi = whole[BAND_BYTES + nbytes:]
        for side, band in (("before", lo), ("after", hi)):
            if not bool((band == PATTERN).all()):
                first = int((band != PATTERN).nonzero()[0])
                off = first - BAND_BYTES if side == "before" else first
                bad.append(f"{name}: the guard band {side} the buffer changed (first damaged byte {off:+d} from the buffer's {'start' if side == 'before' else 'end'})")
    if bad:
        raise CanaryError("; ".join(bad))
    return len(_registry)


def forget(prefix: str = "") -> None:
    """Drops the registered buffers whose name starts with `prefix` (a model that is deleted)."""
    _registry[:] = [r for r in _registry if not r[0].startswith(prefix)]
