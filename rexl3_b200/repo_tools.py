"""Repository-policy tools: the pull-request rules check, the corresponding-source export and the release cut.  Own designs for the roles of
the reference's `tools/check_pr_rules.py`, `tools/build_corresponding_source.py` and `tools/cut_release.py`; everything works on a local git
repository (no hosting API: a CI job passes the title, the branch and the base revision).

    python -m rexl3_b200.repo_tools pr-rules --title "FEAT: Added the burst prefill policy" --branch engine/burst-prefill --base origin/main
    python -m rexl3_b200.repo_tools source-export --commit HEAD --out dist/source.tar.gz
    python -m rexl3_b200.repo_tools cut-release --version v0.2.0            # verification only; --tag also creates the annotated tag locally

Exit status: 0 all rules pass, 1 a rule fails, 2 usage / I/O error, 3 the export was blocked because a private path would have been published.
"""
from __future__ import annotations

import argparse
import gzip
import hashlib
import io
import json
import os
import re
import subprocess
import sys
import tarfile

TYPES = ("FIX", "FEAT", "BUILD", "CI", "TEST", "BUMP", "DOCS")
TITLE_RE = re.compile(r"^(FIX|FEAT|BUILD|CI|TEST|BUMP|DOCS): ([A-Z][a-z]*)( .*)?$")
PAST_IRREGULAR = {"built", "made", "wrote", "rewrote", "split", "set", "ran", "kept", "cut", "put", "found", "held", "led", "left", "read", "sent", "took",
                  "saw", "gave", "brought", "got", "did", "went", "came", "became", "began", "drew", "fell", "felt", "grew", "knew", "met", "paid", "said",
                  "spoke", "stood", "told", "thought", "won"}
NAME_RE = re.compile(r"[a-z0-9][a-z0-9.\-]{0,62}")
VERSION_RE = re.compile(r"v[0-9]+\.[0-9]+\.[0-9]+")
SEALED_RE = re.compile(r"^runtimes/[^/]+/[^/]+/v[1-9][0-9]*/")
FRAGMENTS = "changes/unreleased/"


class ToolError(Exception):
    def __init__(self, message: str, status: int = 2):
        super().__init__(message)
        self.status = status


def _git(repo: str, *args: str, text: bool = True):
    r = subprocess.run(["git", "-C", repo, *args], capture_output=True, text=text)
    if r.returncode != 0:
        err = r.stderr if text else r.stderr.decode("utf-8", "replace")
        raise ToolError(f"git {' '.join(args)}: {err.strip()}")
    return r.stdout


# ====================================================================================================== pull-request rules
def classify_branch(ref):
    """-> (kind, subject) with kind in model | model-approval | engine | release, or (None, reason)."""
    if not isinstance(ref, str) or not ref:
        return None, "branch name missing"
    head, _, rest = ref.partition("/")
    if head == "model":
        if "/" in rest:
            return None, "invalid model branch name"
        if rest.endswith("-approval") and NAME_RE.fullmatch(rest[:-9] or "-"):
            return "model-approval", rest[:-9]
        return ("model", rest) if NAME_RE.fullmatch(rest or "-") else (None, "invalid model branch name")
    if head == "engine":
        return ("engine", rest) if NAME_RE.fullmatch(rest or "-") else (None, "invalid engine topic")
    if head == "release":
        return ("release", rest) if VERSION_RE.fullmatch(rest) else (None, "invalid release branch version")
    return None, "branch is not one of model/<name>, model/<name>-approval, engine/<topic>, release/v<X.Y.Z>"


def title_problems(title) -> list:
    if not isinstance(title, str) or not title.strip():
        return ["title missing"]
    out = []
    if len(title) > 90:
        out.append("title exceeds 90 characters")
    if title.endswith("."):
        out.append("title has a trailing period")
    m = TITLE_RE.fullmatch(title)
    if m is None:
        return out + [f"title is not 'TYPE: Past-tense summary' (TYPE one of {' '.join(TYPES)})"]
    word = m.group(2)
    if not (word.endswith("ed") or word.lower() in PAST_IRREGULAR):
        out.append(f"title verb {word!r} is not past tense")
    return out


def changed_files(repo: str, base: str, head: str = "HEAD") -> list:
    """[(status letter, path)] of base...head (renames reported as delete + add)."""
    out = _git(repo, "diff", "--name-status", "--no-renames", f"{base}...{head}")
    return [tuple(line.split("\t", 1)) for line in out.splitlines() if "\t" in line]


def check_pr_rules(title: str, branch: str, files: list) -> list:
    """-> [(rule, ok, detail)].  files: [(status, path)], status A / M / D."""
    res = []
    kind, subject = classify_branch(branch)
    res.append(("branch", kind is not None, branch if kind else subject))
    probs = title_problems(title)
    res.append(("title", not probs, "; ".join(probs)))
    paths = [p for _, p in files]
    if kind in ("model", "model-approval"):
        outside = [p for p in paths if not re.match(rf"^runtimes/[^/]+/{re.escape(subject)}/", p) and not p.startswith(FRAGMENTS)]
        res.append(("scope", not outside, f"a model branch touches only runtimes/<family>/{subject}/ (and its fragment): {outside[:3]}" if outside else ""))
        if kind == "model-approval":
            other = [p for p in paths if not p.endswith("/approval.json") and not p.endswith("/source.manifest.json") and not p.startswith(FRAGMENTS)]
            res.append(("approval-only", not other, f"an approval branch changes approval.json and the manifest only: {other[:3]}" if other else ""))
    elif kind == "engine":
        sealed = [p for s, p in files if SEALED_RE.match(p) and s != "A"]
        res.append(("sealed-trees", not sealed, f"a sealed recipe version is immutable; add a new version instead: {sealed[:3]}" if sealed else ""))
        rel = [p for p in paths if p.startswith("releases/")]
        res.append(("scope", not rel, f"an engine branch does not touch releases/: {rel[:3]}" if rel else ""))
    elif kind == "release":
        outside = [p for p in paths if not (p.startswith(f"releases/{subject}/") or p == "CHANGELOG.md" or p.startswith(FRAGMENTS))]
        res.append(("scope", not outside, f"a release branch touches releases/{subject}/, CHANGELOG.md and the fragments only: {outside[:3]}" if outside else ""))
    frag_added = [p for s, p in files if p.startswith(FRAGMENTS) and s in ("A", "M")]
    frag_removed = [p for s, p in files if p.startswith(FRAGMENTS) and s == "D"]
    if kind == "release":
        res.append(("fragments", not frag_added, "a release folds the fragments into CHANGELOG.md: it removes them, it adds none" if frag_added else ""))
    elif kind is not None:
        ok = len(frag_added) == 1 and not frag_removed and frag_added[0].endswith(".md")
        res.append(("fragments", ok, "" if ok else f"exactly one changes/unreleased/<topic>.md is added or edited per pull request (found {len(frag_added)}, removed {len(frag_removed)})"))
    return res


# ====================================================================================================== corresponding-source export
EXPORT_SCHEMA = "rexl3-b200.corresponding-source.v1"
EXPORT_ROOTS = ("rexl3_b200/", "tests/", "runtimes/", "dashboard/", "baseline/", "docs/")
EXPORT_FILES = ("bench.py", "__graft_entry__.py", "README.md", "DESIGN.md", "BASELINE.md", ".gitignore")
EXPORT_REQUIRED = ("rexl3_b200/__init__.py", "bench.py", "__graft_entry__.py", "README.md")
PRIVATE_RE = re.compile(r"(^|/)(_work|gpurun_out|\.env|\.ssh|secrets?)(/|$)|\.(pem|key|ncu-rep)$")
MAX_BLOB = 32 << 20
MAX_TOTAL = 256 << 20
MAX_ENTRIES = 20000


def export_source(repo: str, commit: str, out_path: str) -> dict:
    """A deterministic tar.gz of the commit's source: only git objects are read (no checkout, no filters), entries sorted by path, owner,
    group and time zeroed, so the same commit always gives the same bytes.  Fails closed: a required file missing, a blob or the whole over
    its cap, a symlink or submodule inside the exported roots, or (status 3) a path that looks private.  Returns the metadata document,
    also written beside the archive as <out>.json."""
    full = _git(repo, "rev-parse", "--verify", f"{commit}^{{commit}}").strip()
    listing = _git(repo, "ls-tree", "-r", "-z", "--full-tree", "-l", full)
    entries = []
    for rec in listing.split("\0"):
        if not rec:
            continue
        meta, path = rec.split("\t", 1)
        mode, typ, sha, size = meta.split()
        if not (path in EXPORT_FILES or any(path.startswith(r) for r in EXPORT_ROOTS)):
            continue
        if PRIVATE_RE.search(path):
            raise ToolError(f"blocked: {path} looks private and is inside the exported roots", 3)
        if typ != "blob" or mode not in ("100644", "100755"):
            raise ToolError(f"{path}: only regular files are exported (mode {mode}, type {typ})")
        if int(size) > MAX_BLOB:
            raise ToolError(f"{path}: {size} bytes exceeds the {MAX_BLOB}-byte cap")
        entries.append((path, mode, sha, int(size)))
    entries.sort()
    have = {p for p, *_ in entries}
    missing = [p for p in EXPORT_REQUIRED if p not in have]
    if missing:
        raise ToolError(f"the commit lacks required files: {missing}")
    if len(entries) > MAX_ENTRIES or sum(e[3] for e in entries) > MAX_TOTAL:
        raise ToolError("the export exceeds its entry or size cap")
    raw = io.BytesIO()
    files = {}
    with tarfile.open(fileobj=raw, mode="w", format=tarfile.PAX_FORMAT) as tar:
        for path, mode, sha, size in entries:
            data = _git(repo, "cat-file", "blob", sha, text=False)
            if len(data) != size:
                raise ToolError(f"{path}: object size changed while reading")
            info = tarfile.TarInfo(f"rexl3-b200-{full[:12]}/{path}")
            info.size, info.mode, info.mtime, info.uid, info.gid, info.uname, info.gname = size, 0o755 if mode == "100755" else 0o644, 0, 0, 0, "", ""
            tar.addfile(info, io.BytesIO(data))
            files[path] = {"sha256": hashlib.sha256(data).hexdigest(), "bytes": size}
    packed = io.BytesIO()
    with gzip.GzipFile(fileobj=packed, mode="wb", mtime=0, compresslevel=9) as gz:
        gz.write(raw.getvalue())
    blob = packed.getvalue()
    os.makedirs(os.path.dirname(os.path.abspath(out_path)), exist_ok=True)
    with open(out_path, "wb") as f:
        f.write(blob)
    doc = {"schema": EXPORT_SCHEMA, "commit": full, "archive": os.path.basename(out_path), "archive_sha256": hashlib.sha256(blob).hexdigest(),
           "archive_bytes": len(blob), "files": files}
    with open(out_path + ".json", "w", encoding="utf-8") as f:
        json.dump(doc, f, indent=1, sort_keys=True)
        f.write("\n")
    return doc


# ====================================================================================================== release cut
def cut_release(repo: str, version: str, tag: bool = False) -> list:
    """The gates of a release, all evaluated: -> [(gate, ok, detail)].  With tag=True and every gate green, an annotated tag is created locally
    (never pushed: publishing is a maintainer's step)."""
    res = []
    ok_v = bool(VERSION_RE.fullmatch(version or ""))
    res.append(("version", ok_v, "" if ok_v else "version must look like v<X>.<Y>.<Z>"))
    if not ok_v:
        return res
    tags = _git(repo, "tag", "-l", version).split()
    res.append(("tag-absent", version not in tags, "" if version not in tags else f"tag {version} exists already"))
    dirty = _git(repo, "status", "--porcelain", "--untracked-files=no").strip()
    res.append(("clean-tree", not dirty, "" if not dirty else "tracked files have uncommitted changes"))
    notes = os.path.join(repo, "releases", version, "NOTES.md")
    res.append(("notes", os.path.isfile(notes) and os.path.getsize(notes) > 0, "" if os.path.isfile(notes) else f"releases/{version}/NOTES.md is missing"))
    cl = os.path.join(repo, "CHANGELOG.md")
    has = os.path.isfile(cl) and re.search(rf"^## {re.escape(version)}\b", open(cl, encoding="utf-8").read(), re.M) is not None
    res.append(("changelog", has, "" if has else f"CHANGELOG.md has no '## {version}' entry"))
    frdir = os.path.join(repo, "changes", "unreleased")
    left = sorted(n for n in os.listdir(frdir) if n.endswith(".md")) if os.path.isdir(frdir) else []
    res.append(("fragments-folded", not left, "" if not left else f"unreleased fragments remain: {left[:3]}"))
    from . import release
    rt = os.path.join(repo, "runtimes")
    bad = release.verify_all(rt) if os.path.isdir(rt) else ["no runtimes/ directory"]
    res.append(("recipes", not bad, "" if not bad else "; ".join(bad[:3])))
    if tag and all(ok for _, ok, _ in res):
        _git(repo, "tag", "-a", version, "-m", f"rexl3-b200 {version}")
        res.append(("tag-created", True, version))
    return res


def _report(results, out) -> int:
    for name, ok, detail in results:
        print(f"{'PASS' if ok else 'FAIL'} {name}{': ' + detail if detail else ''}", file=out)
    return 0 if all(ok for _, ok, _ in results) else 1


def main(argv=None, out=sys.stdout) -> int:
    p = argparse.ArgumentParser(prog="rexl3-repo-tools", allow_abbrev=False)
    sub = p.add_subparsers(dest="cmd", required=True)
    a = sub.add_parser("pr-rules")
    a.add_argument("--title", required=True)
    a.add_argument("--branch", required=True)
    a.add_argument("--base", required=True, help="base revision; the changed files are base...HEAD")
    a.add_argument("--head", default="HEAD")
    a.add_argument("--repo", default=".")
    b = sub.add_parser("source-export")
    b.add_argument("--commit", default="HEAD")
    b.add_argument("--out", required=True)
    b.add_argument("--repo", default=".")
    c = sub.add_parser("cut-release")
    c.add_argument("--version", required=True)
    c.add_argument("--tag", action="store_true")
    c.add_argument("--repo", default=".")
    args = p.parse_args(argv)
    try:
        if args.cmd == "pr-rules":
            return _report(check_pr_rules(args.title, args.branch, changed_files(args.repo, args.base, args.head)), out)
        if args.cmd == "source-export":
            doc = export_source(args.repo, args.commit, args.out)
            print(f"{doc['archive']} {doc['archive_bytes']} bytes sha256 {doc['archive_sha256']} ({len(doc['files'])} files of {doc['commit'][:12]})", file=out)
            return 0
        return _report(cut_release(args.repo, args.version, args.tag), out)
    except ToolError as e:
        print(f"rexl3-repo-tools: {e}", file=sys.stderr)
        return e.status


if __name__ == "__main__":
    sys.exit(main())
