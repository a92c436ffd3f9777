"""Recipe trees: `runtimes/<family>/<model>/{MODEL.json, LATEST, v<N>/{profile.json, approval.json, model.lock.json, launch.sh, ...}}`.

A profile names an argv template for the serving binary with `@SITE_FIELD@` placeholders (`@MODEL_DIR@`, `@HTTP_PORT@`, ...); a site
file supplies the fields.  `resolve` picks the version (LATEST unless given), the profile (default_profile unless given), renders
the argv, and refuses: a missing site field, a placeholder left unrendered, a flag the serving binary does not know (so a recipe
written for another build fails at load time, not at 3 a.m.), a profile whose state is not "final" unless `allow_draft`.
Layout parity: reference README.md:186-210 and runtimes/qwen3.8/qwen3.8-27b/v4/profile.json (schema rexl3.runtime-profile.v1).
"""
from __future__ import annotations

import json
import os
import re
from dataclasses import dataclass, field

PROFILE_SCHEMA = "rexl3.runtime-profile.v1"
MODEL_SCHEMA = "rexl3.prod-model.v1"


class RecipeError(ValueError):
    pass


@dataclass
class Resolved:
    runtime_id: str
    version: str
    profile: str
    argv: list
    env: dict = field(default_factory=dict)
    capabilities: dict = field(default_factory=dict)
    smoke_request: dict | None = None
    readiness_timeout_s: int = 600
    http_host: str = "127.0.0.1"
    http_port: int = 8000
    kind: str = "single"            # "single" | "tp" (one process per GPU under torch.distributed.run)
    ranks: int = 1
    rendezvous_port: int = 29540
    model_dir: str | None = None


def _read_json(path):
    try:
        with open(path) as f:
            return json.load(f)
    except OSError as e:
        raise RecipeError(f"{path}: {e.strerror}") from e
    except json.JSONDecodeError as e:
        raise RecipeError(f"{path}: {e}") from e


def known_flags() -> set:
    from .server.main import parser
    out = set()
    for a in parser()._actions:
        out.update(o for o in a.option_strings if o.startswith("--"))
    return out


def resolve(root: str, family: str, model: str, site: dict, version: str | None = None, profile: str | None = None, allow_draft: bool = False,
            check_flags: bool = True) -> Resolved:
    base = os.path.join(root, family, model)
    meta = _read_json(os.path.join(base, "MODEL.json"))
    if meta.get("schema") != MODEL_SCHEMA:
        raise RecipeError(f"{base}/MODEL.json: schema {meta.get('schema')!r}, expected {MODEL_SCHEMA!r}")
    if version is None:
        try:
            version = open(os.path.join(base, "LATEST")).read().strip()
        except OSError as e:
            raise RecipeError(f"{base}/LATEST: {e.strerror}") from e
    if not re.fullmatch(r"v\d+", version):
        raise RecipeError(f"bad version {version!r}")
    vdir = os.path.join(base, version)
    doc = _read_json(os.path.join(vdir, "profile.json"))
    if doc.get("schema") != PROFILE_SCHEMA:
        raise RecipeError(f"{vdir}/profile.json: schema {doc.get('schema')!r}, expected {PROFILE_SCHEMA!r}")
    if doc.get("runtime_id") != meta.get("runtime_id"):
        raise RecipeError(f"runtime_id differs between MODEL.json ({meta.get('runtime_id')!r}) and {version}/profile.json ({doc.get('runtime_id')!r})")
    if doc.get("state") != "final" and not allow_draft:
        raise RecipeError(f"{version}/profile.json is in state {doc.get('state')!r}, not 'final'")
    name = profile or doc.get("default_profile")
    prof = (doc.get("profiles") or {}).get(name)
    if prof is None:
        raise RecipeError(f"profile {name!r} is not in {version}/profile.json (has: {sorted(doc.get('profiles') or {})})")
    fields = {**{k: prof[k] for k in ("http_host", "http_port") if k in prof}, **site}
    missing = [f for f in prof.get("site_fields", []) if f not in fields]
    if missing:
        raise RecipeError(f"site file lacks: {missing}")
    argv = []
    for a in prof.get("argv", []):
        for k, v in fields.items():
            a = a.replace(f"@{k.upper()}@", str(v))
        left = re.findall(r"@[A-Z_]+@", a)
        if left:
            raise RecipeError(f"unrendered placeholder {left[0]} (no site field for it)")
        argv.append(a)
    if check_flags:
        flags = known_flags()
        unknown = [a for a in argv if a.startswith("--") and a.split("=")[0] not in flags]
        if unknown:
            raise RecipeError(f"flags this serving binary does not know: {unknown}")
    return Resolved(doc["runtime_id"], version, name, argv, dict(prof.get("env", {})), dict(prof.get("capabilities", {})), prof.get("smoke_request"),
                    int(prof.get("readiness_timeout_s", 600)), str(fields.get("http_host", "127.0.0.1")), int(fields.get("http_port", 8000)),
                    str(prof.get("kind", "single")), int(prof.get("ranks", 1)), int(prof.get("rendezvous_port", 29540)), fields.get("model_dir"))


def seal(vdir: str) -> dict:
    """Write `source.manifest.json` of a recipe version directory: the sha256 and size of every file in it (the manifest itself excluded)."""
    import hashlib
    files = {}
    for base, _dirs, names in os.walk(vdir):
        for n in sorted(names):
            path = os.path.join(base, n)
            rel = os.path.relpath(path, vdir)
            if rel == "source.manifest.json":
                continue
            with open(path, "rb") as f:
                data = f.read()
            files[rel] = {"sha256": hashlib.sha256(data).hexdigest(), "bytes": len(data)}
    doc = {"schema": "rexl3.source-manifest.v1", "files": files}
    with open(os.path.join(vdir, "source.manifest.json"), "w") as f:
        json.dump(doc, f, indent=1, sort_keys=True)
        f.write("\n")
    return doc


def verify_tree(vdir: str) -> list:
    """Problems of a sealed recipe version directory against its manifest: missing, changed and unlisted files.  Empty list: intact.
    (What the reference's tools/verify_runtime_tree.py checks for its sealed trees.)"""
    import hashlib
    doc = _read_json(os.path.join(vdir, "source.manifest.json"))
    if doc.get("schema") != "rexl3.source-manifest.v1" or not isinstance(doc.get("files"), dict):
        raise RecipeError(f"{vdir}/source.manifest.json: not a source manifest")
    problems = []
    seen = set()
    for rel, want in sorted(doc["files"].items()):
        path = os.path.join(vdir, rel)
        seen.add(rel)
        if not os.path.isfile(path):
            problems.append(f"missing: {rel}")
            continue
        with open(path, "rb") as f:
            data = f.read()
        if hashlib.sha256(data).hexdigest() != want.get("sha256") or len(data) != want.get("bytes"):
            problems.append(f"changed: {rel}")
    for base, _dirs, names in os.walk(vdir):
        for n in names:
            rel = os.path.relpath(os.path.join(base, n), vdir)
            if rel != "source.manifest.json" and rel not in seen:
                problems.append(f"unlisted: {rel}")
    return problems


def main(argv=None) -> int:
    import argparse
    import shlex
    import sys
    p = argparse.ArgumentParser(prog="rexl3-recipe", allow_abbrev=False)
    p.add_argument("--root", default="runtimes")
    p.add_argument("--family", required=True)
    p.add_argument("--model", required=True)
    p.add_argument("--site", required=True, help="JSON file of site fields (model_dir, http_port, ...)")
    p.add_argument("--version")
    p.add_argument("--profile")
    p.add_argument("--exec", action="store_true", help="exec the serving binary instead of printing the command")
    p.add_argument("--verify", action="store_true", help="check the version directory against its source manifest first; refuse a changed tree")
    a = p.parse_args(argv)
    if a.verify:
        try:
            version = a.version or open(os.path.join(a.root, a.family, a.model, "LATEST")).read().strip()
            problems = verify_tree(os.path.join(a.root, a.family, a.model, version))
        except (RecipeError, OSError) as e:
            print(f"rexl3-recipe: {e}", file=sys.stderr)
            return 2
        if problems:
            print("rexl3-recipe: the sealed tree does not match its manifest:\n  " + "\n  ".join(problems), file=sys.stderr)
            return 2
    try:
        r = resolve(a.root, a.family, a.model, _read_json(a.site), a.version, a.profile)
    except RecipeError as e:
        print(f"rexl3-recipe: {e}", file=sys.stderr)
        return 2
    cmd = [sys.executable, "-m", "rexl3_b200.server"] + r.argv
    if a.exec:
        os.execvpe(cmd[0], cmd, {**os.environ, **r.env})
    print(" ".join(shlex.quote(c) for c in cmd))
    return 0


if __name__ == "__main__":
    import sys
    sys.exit(main())
