"""``python -m rexl3_b200.format.inspect_cli DIR`` - what a pack holds, without reading tensor data: every EXL3 group (shape, bits,
codebook, bytes), the plain tensors, the refusals by name, the overall bits per weight.  Exit status 0 when every group parses
and no header issue was found, 1 otherwise.  Counterpart of the reference's `exl3-inspect` (crates/exl3/src/bin)."""
from __future__ import annotations

import argparse
import json
import sys

from .checkpoint import scan


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="exl3-inspect", allow_abbrev=False)
    p.add_argument("folder")
    p.add_argument("--json", action="store_true")
    p.add_argument("--groups", action="store_true", help="list every group (default: a summary by bit width)")
    a = p.parse_args(argv)
    ck = scan(a.folder)
    weights = sum(g.k * g.n for g in ck.groups.values())
    tbytes = sum(g.bytes for g in ck.groups.values())
    by_bits = {}
    for g in ck.groups.values():
        k = f"{g.bits.value:g}/{g.codebook}"
        e = by_bits.setdefault(k, [0, 0])
        e[0] += 1
        e[1] += g.k * g.n
    doc = {"folder": a.folder, "groups": len(ck.groups), "plain_tensors": len(ck.plain), "bad_groups": ck.bad, "issues": ck.issues,
           "weights": weights, "bytes": ck.total_bytes(), "bits_per_weight": round(8 * tbytes / weights, 4) if weights else None,
           "by_bits": {k: {"groups": v[0], "weights": v[1]} for k, v in sorted(by_bits.items())}}
    if a.groups:
        doc["group_list"] = [dict(prefix=g.prefix, k=g.k, n=g.n, bits=g.bits.value, codebook=g.codebook, bias=g.bias, bytes=g.bytes) for g in ck.groups.values()]
    if a.json:
        print(json.dumps(doc))
    else:
        print(f"{a.folder}: {doc['groups']} EXL3 groups, {doc['plain_tensors']} plain tensors, {doc['bytes'] / 1e9:.3f} GB, "
              f"{doc['bits_per_weight']} bits per weight")
        for k, v in doc["by_bits"].items():
            print(f"  {k:>12}: {v['groups']:5d} groups, {v['weights'] / 1e6:10.1f} M weights")
        for g in doc.get("group_list", []):
            print(f"  {g['prefix']}: [{g['k']}, {g['n']}] {g['bits']:g} bpw {g['codebook']}{' +bias' if g['bias'] else ''}")
        for pre, why in ck.bad.items():
            print(f"  REFUSED {pre}: {why}")
        for i in ck.issues:
            print(f"  ISSUE {i}")
    return 0 if not ck.bad and not ck.issues else 1


if __name__ == "__main__":
    sys.exit(main())
