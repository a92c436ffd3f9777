"""Release governance over the recipe trees: check every sealed tree, promote a version to LATEST, collect release evidence.

Roles (reference `tools/verify_runtime_tree.py`, `tools/promote_runtime.py`, `tools/release_evidence.py`):
  verify-all   every `runtimes/<family>/<model>/<version>` is intact against its manifest, its profile resolves with a sample site and
               names only flags the serving binary has, and LATEST points at an existing, final, approved version;
  promote      make a version the LATEST one: refused unless the tree is sealed and intact, the profile state is "final" and
               `approval.json` in the version directory says who approved it (the approval is part of the sealed tree);
  evidence     one JSON document for a release: per recipe the version, manifest digest and approval; the git revision; the kernel
               library's hash; the measured numbers found in the repository's BENCH / SCALE JSON files, if any.

    python -m rexl3_b200.release verify-all
    python -m rexl3_b200.release promote --family dense --model dense-27b --version v2
    python -m rexl3_b200.release evidence --out release-evidence.json
"""
from __future__ import annotations

import glob
import hashlib
import json
import os
import subprocess
import sys

from . import recipes

SAMPLE_SITE = {"http_host": "127.0.0.1", "http_port": 8000, "model_dir": "/models/sample", "spill_dir": "/nvme/spill", "tp_port": 29600}


def _trees(root: str):
    for fam in sorted(os.listdir(root)):
        fdir = os.path.join(root, fam)
        if not os.path.isdir(fdir):
            continue
        for model in sorted(os.listdir(fdir)):
            mdir = os.path.join(fdir, model)
            if os.path.isfile(os.path.join(mdir, "MODEL.json")):
                yield fam, model, mdir


def _versions(mdir: str) -> list:
    return sorted((v for v in os.listdir(mdir) if v.startswith("v") and v[1:].isdigit() and os.path.isdir(os.path.join(mdir, v))), key=lambda v: int(v[1:]))


def approval_of(vdir: str):
    p = os.path.join(vdir, "approval.json")
    if not os.path.isfile(p):
        return None
    try:
        a = json.load(open(p))
    except ValueError:
        return None
    return a if a.get("approved") is True and a.get("approved_by") else None


def verify_all(root: str = "runtimes") -> list:
    problems = []
    for fam, model, mdir in _trees(root):
        tag = f"{fam}/{model}"
        vs = _versions(mdir)
        if not vs:
            problems.append(f"{tag}: no version directory")
            continue
        try:
            latest = open(os.path.join(mdir, "LATEST")).read().strip()
        except OSError:
            problems.append(f"{tag}: no LATEST")
            latest = None
        if latest is not None and latest not in vs:
            problems.append(f"{tag}: LATEST names {latest!r}, which does not exist")
        for v in vs:
            vdir = os.path.join(mdir, v)
            try:
                problems += [f"{tag}/{v}: {p}" for p in recipes.verify_tree(vdir)]
            except recipes.RecipeError as e:
                problems.append(f"{tag}/{v}: {e}")
            try:
                prof = json.load(open(os.path.join(vdir, "profile.json")))
                for name in prof.get("profiles", {}):
                    recipes.resolve(root, fam, model, SAMPLE_SITE, v, name, allow_draft=True)
            except (recipes.RecipeError, OSError, ValueError) as e:
                problems.append(f"{tag}/{v}: {e}")
                continue
            if v == latest:
                if prof.get("state") != "final":
                    problems.append(f"{tag}/{v}: LATEST points at a profile in state {prof.get('state')!r}")
                if approval_of(vdir) is None:
                    problems.append(f"{tag}/{v}: LATEST points at a version without an approval")
    return problems


def promote(root: str, family: str, model: str, version: str) -> str:
    mdir = os.path.join(root, family, model)
    vdir = os.path.join(mdir, version)
    if not os.path.isdir(vdir):
        raise recipes.RecipeError(f"{family}/{model}/{version}: no such version")
    bad = recipes.verify_tree(vdir)
    if bad:
        raise recipes.RecipeError(f"{family}/{model}/{version}: the tree does not match its manifest ({bad[0]})")
    prof = json.load(open(os.path.join(vdir, "profile.json")))
    if prof.get("state") != "final":
        raise recipes.RecipeError(f"{family}/{model}/{version}: profile state is {prof.get('state')!r}, not 'final'")
    if approval_of(vdir) is None:
        raise recipes.RecipeError(f"{family}/{model}/{version}: approval.json with approved=true and approved_by is required")
    for name in prof.get("profiles", {}):
        recipes.resolve(root, family, model, SAMPLE_SITE, version, name)
    tmp = os.path.join(mdir, "LATEST.tmp")
    with open(tmp, "w") as f:
        f.write(version + "\n")
    os.replace(tmp, os.path.join(mdir, "LATEST"))
    return version


def _git_rev(repo: str):
    try:
        r = subprocess.run(["git", "-C", repo, "rev-parse", "HEAD"], capture_output=True, text=True, timeout=10)
        return r.stdout.strip() or None
    except (OSError, subprocess.SubprocessError):
        return None


def evidence(root: str = "runtimes", repo: str = ".") -> dict:
    out = {"schema": "rexl3.release-evidence.v1", "git_revision": _git_rev(repo), "recipes": [], "measurements": [], "problems": verify_all(root)}
    for fam, model, mdir in _trees(root):
        try:
            latest = open(os.path.join(mdir, "LATEST")).read().strip()
        except OSError:
            continue
        vdir = os.path.join(mdir, latest)
        man = os.path.join(vdir, "source.manifest.json")
        out["recipes"].append({"family": fam, "model": model, "version": latest,
                               "manifest_sha256": hashlib.sha256(open(man, "rb").read()).hexdigest() if os.path.isfile(man) else None,
                               "approval": approval_of(vdir)})
    from .ops import lib as oplib
    if os.path.exists(oplib.LIB_PATH):
        out["kernel_library_sha256"] = hashlib.sha256(open(oplib.LIB_PATH, "rb").read()).hexdigest()
    for path in sorted(glob.glob(os.path.join(repo, "BENCH_r*.json")) + glob.glob(os.path.join(repo, "SCALE_r*.json"))):
        try:
            out["measurements"].append({"file": os.path.basename(path), "data": json.load(open(path))})
        except (OSError, ValueError):
            pass
    return out


def main(argv=None) -> int:
    import argparse
    p = argparse.ArgumentParser(prog="rexl3-release", allow_abbrev=False)
    p.add_argument("command", choices=["verify-all", "promote", "evidence"])
    p.add_argument("--root", default="runtimes")
    p.add_argument("--family")
    p.add_argument("--model")
    p.add_argument("--version")
    p.add_argument("--out", default="")
    a = p.parse_args(argv)
    if a.command == "verify-all":
        bad = verify_all(a.root)
        for b in bad:
            print("PROBLEM", b)
        print("ok" if not bad else f"{len(bad)} problems")
        return 1 if bad else 0
    if a.command == "promote":
        if not (a.family and a.model and a.version):
            print("rexl3-release: promote needs --family, --model and --version", file=sys.stderr)
            return 2
        try:
            print("LATEST ->", promote(a.root, a.family, a.model, a.version))
            return 0
        except (recipes.RecipeError, OSError, ValueError) as e:
            print(f"rexl3-release: refused: {e}", file=sys.stderr)
            return 2
    doc = evidence(a.root, os.path.dirname(os.path.abspath(a.root)) or ".")
    text = json.dumps(doc, indent=1, sort_keys=True)
    if a.out:
        open(a.out, "w").write(text + "\n")
    else:
        print(text)
    return 1 if doc["problems"] else 0


if __name__ == "__main__":
    sys.exit(main())
