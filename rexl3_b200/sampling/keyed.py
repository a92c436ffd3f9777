"""Keyed Gumbel sampler: the token at absolute position p is a pure function of (logits row, seed, p).

token = argmax over the kept candidates of logit/T + Gumbel(splitmix64(seed, p, id)); T == 0 is argmax with
ties to the lowest id.  All arithmetic is float64 in numpy's order (pairwise sum for the softmax total) so the
choice matches the reference bit for bit (crates/sampling/src/lib.rs:94-150 hashing, :152-182 pairwise sum,
:210-268 choose, :284-300 top candidates).  A speculative draft is accepted iff it equals this sample, which is
what makes speculation change speed and never an output byte.
"""
from __future__ import annotations

import hashlib
import math
from dataclasses import dataclass, replace

import numpy as np

MARGIN = 8  # candidates read beyond top_k so ties at the cut resolve by id
_M = 0xFFFFFFFFFFFFFFFF
TWO_M53 = 1.0 / 9007199254740992.0
TWO_M54 = TWO_M53 / 2.0
BELOW_ONE = 1.0 - TWO_M53


class SamplingError(ValueError):
    pass


@dataclass(frozen=True)
class Sampling:
    seed: int = 0
    temperature: float = 1.0
    top_k: int = 20
    top_p: float = 0.95
    min_p: float = 0.0

    def candidate_count(self, vocab: int) -> int:
        return vocab if self.top_k == 0 else min(self.top_k + MARGIN, vocab)

    def validate(self) -> None:
        if not math.isfinite(self.temperature) or self.temperature < 0.0:
            raise SamplingError("invalid sampling parameters: temperature must be finite and >= 0")
        if not math.isfinite(self.top_p) or not 0.0 <= self.top_p <= 1.0:
            raise SamplingError("invalid sampling parameters: top_p must be in [0, 1]")
        if not math.isfinite(self.min_p) or not 0.0 <= self.min_p <= 1.0:
            raise SamplingError("invalid sampling parameters: min_p must be in [0, 1]")

    def with_seed(self, seed: int) -> "Sampling":
        return replace(self, seed=seed)


GREEDY = Sampling(seed=0, temperature=0.0, top_k=1, top_p=1.0, min_p=0.0)


def seed_for(tokens, salt: int = 0) -> int:
    """sha256("t0,t1,...|salt")[:8] little-endian with the top bit cleared: same conversation, same reply."""
    h = hashlib.sha256()
    h.update(",".join(str(int(t)) for t in tokens).encode())
    h.update(b"|")
    h.update(str(int(salt)).encode())
    return int.from_bytes(h.digest()[:8], "little") & ((1 << 63) - 1)


def _mix(x: int) -> int:
    x ^= x >> 30
    x = (x * 0xBF58476D1CE4E5B9) & _M
    x ^= x >> 27
    x = (x * 0x94D049BB133111EB) & _M
    return x ^ (x >> 31)


def unit_open(x: int) -> float:
    return min((x >> 11) * TWO_M53 + TWO_M54, BELOW_ONE)


def uniform(seed: int, position: int, tid: int) -> float:
    x = _mix((seed + 0x9E3779B97F4A7C15) & _M)
    x = _mix(x ^ ((position * 0xD1B54A32D192ED03) & _M))
    x = _mix(x ^ (tid & _M))
    return unit_open(x)


def gumbel(seed: int, position: int, tid: int) -> float:
    return -math.log(-math.log(uniform(seed, position, tid)))


def pairwise_sum(a) -> float:
    """numpy's float64 pairwise summation of a contiguous array."""
    n = len(a)
    if n < 8:
        r = 0.0
        for v in a:
            r += v
        return r
    if n <= 128:
        r = [a[j] for j in range(8)]
        i = 8
        while i < n - (n % 8):
            for j in range(8):
                r[j] += a[i + j]
            i += 8
        res = ((r[0] + r[1]) + (r[2] + r[3])) + ((r[4] + r[5]) + (r[6] + r[7]))
        while i < n:
            res += a[i]
            i += 1
        return res
    n2 = n // 2
    n2 -= n2 % 8
    return pairwise_sum(a[:n2]) + pairwise_sum(a[n2:])


def choose(values, ids, position: int, s: Sampling) -> int:
    """One row: candidate logits ``values`` (float32) for token ``ids`` at absolute ``position`` -> token id."""
    s.validate()
    values = [float(np.float32(v)) for v in values]
    ids = [int(i) for i in ids]
    if len(values) != len(ids):
        raise SamplingError(f"{len(values)} logits but {len(ids)} candidate ids")
    if not values:
        raise SamplingError("no candidates")
    if any(v != v for v in values):
        raise SamplingError("NaN logit")
    if s.temperature == 0.0:
        best = 0
        for i in range(1, len(values)):
            if values[i] > values[best] or (values[i] == values[best] and ids[i] < ids[best]):
                best = i
        return ids[best]
    order = sorted(range(len(values)), key=lambda i: (-values[i], ids[i]))
    n = len(ids)
    k = max(min(s.top_k, n) if s.top_k > 0 else n, 1)
    t = max(s.temperature, 1e-6)
    kid = [ids[i] for i in order[:k]]
    scaled = [values[i] / t for i in order[:k]]
    if 0.0 < s.top_p < 1.0:
        mx = max(scaled)
        probs = [math.exp(v - mx) for v in scaled]
        total = pairwise_sum(probs)
        probs = [p / total for p in probs]
        c, below = 0.0, 0
        for p in probs:
            c += p
            if c < s.top_p:
                below += 1
        keep = min(below + 1, k)
        kid, scaled = kid[:keep], scaled[:keep]
    if s.min_p > 0.0:
        floor = scaled[0] + math.log(s.min_p)
        keep = max(sum(1 for v in scaled if v >= floor), 1)
        kid, scaled = kid[:keep], scaled[:keep]
    best, best_score = 0, -math.inf
    for i, (tid, v) in enumerate(zip(kid, scaled)):
        score = v + gumbel(s.seed, position, tid)
        if score > best_score:
            best_score, best = score, i
    return kid[best]


def choose_rows(values, ids, positions, s: Sampling):
    if not (len(values) == len(ids) == len(positions)):
        raise SamplingError("choose_rows: values, ids and positions differ in length")
    return [choose(v, i, p, s) for v, i, p in zip(values, ids, positions)]


def top_candidates(logits, count: int):
    """Exact top-``count`` of a full logits row ordered (value desc, id asc)."""
    logits = np.asarray(logits, dtype=np.float32)
    if np.isnan(logits).any():
        raise SamplingError("NaN logit")
    take = min(count, logits.shape[0])
    idx = np.lexsort((np.arange(logits.shape[0]), -logits.astype(np.float64)))[:take]
    return idx.astype(np.uint32), logits[idx]
