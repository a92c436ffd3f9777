"""Pull-request rules, the deterministic source export and the release gates, on throw-away git repositories."""
import hashlib
import io
import json
import os
import subprocess
import tarfile

import pytest

from rexl3_b200 import repo_tools as T


def git(repo, *args):
    subprocess.run(["git", "-C", str(repo), *args], check=True, capture_output=True)


@pytest.fixture()
def repo(tmp_path):
    r = tmp_path / "repo"
    r.mkdir()
    git(r, "init", "-q", "-b", "main")
    git(r, "config", "user.email", "t@example.invalid")
    git(r, "config", "user.name", "t")
    for path, text in {"rexl3_b200/__init__.py": "", "bench.py": "print(1)\n", "__graft_entry__.py": "\n", "README.md": "# x\n", "tests/test_a.py": "\n",
                       "docs/notes.md": "n\n", "scratch.txt": "not exported\n"}.items():
        f = r / path
        f.parent.mkdir(parents=True, exist_ok=True)
        f.write_text(text)
    git(r, "add", "-A")
    git(r, "commit", "-q", "-m", "base")
    return r


def test_branch_and_title_rules():
    assert T.classify_branch("engine/burst-prefill") == ("engine", "burst-prefill")
    assert T.classify_branch("model/dense-27b-approval") == ("model-approval", "dense-27b")
    assert T.classify_branch("release/v1.2.3") == ("release", "v1.2.3")
    assert T.classify_branch("feature/x")[0] is None and T.classify_branch("release/1.2")[0] is None and T.classify_branch("model/a/b")[0] is None
    assert T.title_problems("FEAT: Added the burst prefill policy") == []
    assert T.title_problems("FIX: Rewrote the epilogue") == []
    assert any("past tense" in p for p in T.title_problems("FEAT: Add the policy"))
    assert any("trailing period" in p for p in T.title_problems("DOCS: Updated the notes."))
    assert T.title_problems("added stuff") and T.title_problems("") == ["title missing"] and T.title_problems("FEAT: " + "Added " + "x" * 90)


def test_scope_sealed_tree_and_fragment_rules():
    ok = [("M", "rexl3_b200/engine/core.py"), ("A", "changes/unreleased/burst.md")]
    assert all(o for _, o, _ in T.check_pr_rules("FEAT: Added the burst policy", "engine/burst", ok))
    res = dict((n, (o, d)) for n, o, d in T.check_pr_rules("FEAT: Added the burst policy", "engine/burst",
                                                           ok + [("M", "runtimes/dense/dense-27b/v1/profile.json")]))
    assert not res["sealed-trees"][0] and "immutable" in res["sealed-trees"][1]
    newv = ok + [("A", "runtimes/dense/dense-27b/v2/profile.json")]
    assert all(o for _, o, _ in T.check_pr_rules("FEAT: Added the burst policy", "engine/burst", newv))          # a NEW version is an addition
    assert not dict((n, o) for n, o, _ in T.check_pr_rules("FEAT: Added x", "engine/x", [("M", "a.py")]))["fragments"]
    m = T.check_pr_rules("BUMP: Tuned the window rows", "model/dense-27b", [("A", "runtimes/dense/dense-27b/v2/profile.json"), ("M", "rexl3_b200/x.py"),
                                                                            ("A", "changes/unreleased/d.md")])
    assert not dict((n, o) for n, o, _ in m)["scope"]
    ap = T.check_pr_rules("BUMP: Approved the profile", "model/dense-27b-approval", [("M", "runtimes/dense/dense-27b/v2/approval.json"),
                                                                                  ("M", "runtimes/dense/dense-27b/v2/source.manifest.json"), ("A", "changes/unreleased/a.md")])
    assert all(o for _, o, _ in ap)
    rel = T.check_pr_rules("DOCS: Released the version", "release/v0.2.0", [("A", "releases/v0.2.0/NOTES.md"), ("M", "CHANGELOG.md"), ("D", "changes/unreleased/a.md")])
    assert all(o for _, o, _ in rel)
    rel_bad = T.check_pr_rules("DOCS: Released the version", "release/v0.2.0", [("A", "releases/v0.2.0/NOTES.md"), ("A", "changes/unreleased/b.md"), ("M", "bench.py")])
    d = dict((n, o) for n, o, _ in rel_bad)
    assert not d["scope"] and not d["fragments"]


def test_pr_rules_cli_reads_the_diff(repo):
    git(repo, "checkout", "-q", "-b", "engine/topic")
    (repo / "rexl3_b200" / "new.py").write_text("x = 1\n")
    (repo / "changes" / "unreleased").mkdir(parents=True)
    (repo / "changes" / "unreleased" / "topic.md").write_text("- new\n")
    git(repo, "add", "-A")
    git(repo, "commit", "-q", "-m", "topic")
    out = io.StringIO()
    assert T.main(["pr-rules", "--title", "FEAT: Added a module", "--branch", "engine/topic", "--base", "main", "--repo", str(repo)], out=out) == 0
    assert "PASS fragments" in out.getvalue()
    out = io.StringIO()
    assert T.main(["pr-rules", "--title", "Add a module", "--branch", "engine/topic", "--base", "main", "--repo", str(repo)], out=out) == 1
    assert "FAIL title" in out.getvalue()


def test_source_export_is_deterministic_and_fails_closed(repo, tmp_path):
    a = T.export_source(str(repo), "HEAD", str(tmp_path / "a" / "src.tar.gz"))
    b = T.export_source(str(repo), "HEAD", str(tmp_path / "b" / "src.tar.gz"))
    assert a["archive_sha256"] == b["archive_sha256"] and a["files"] == b["files"]
    assert "scratch.txt" not in a["files"] and "docs/notes.md" in a["files"] and "bench.py" in a["files"]
    data = (tmp_path / "a" / "src.tar.gz").read_bytes()
    assert hashlib.sha256(data).hexdigest() == a["archive_sha256"]
    with tarfile.open(fileobj=io.BytesIO(data)) as tar:
        names = tar.getnames()
        assert names == sorted(names) and all(m.mtime == 0 and m.uid == 0 for m in tar.getmembers())
        inner = tar.extractfile(next(n for n in names if n.endswith("/bench.py"))).read()
    assert inner == b"print(1)\n" and json.load(open(tmp_path / "a" / "src.tar.gz.json"))["commit"] == a["commit"]
    # a private-looking path inside the exported roots blocks the export (status 3), a missing required file refuses it (status 2)
    (repo / "rexl3_b200" / "_work").mkdir()
    (repo / "rexl3_b200" / "_work" / "probe.py").write_text("x\n")
    git(repo, "add", "-A")
    git(repo, "commit", "-q", "-m", "oops")
    with pytest.raises(T.ToolError) as e:
        T.export_source(str(repo), "HEAD", str(tmp_path / "c.tar.gz"))
    assert e.value.status == 3
    git(repo, "rm", "-q", "-r", "rexl3_b200/_work", "bench.py")
    git(repo, "commit", "-q", "-m", "no bench")
    with pytest.raises(T.ToolError) as e:
        T.export_source(str(repo), "HEAD", str(tmp_path / "d.tar.gz"))
    assert e.value.status == 2 and "bench.py" in str(e.value)
    os.symlink("README.md", repo / "docs" / "link.md")
    (repo / "bench.py").write_text("x\n")
    git(repo, "add", "-A")
    git(repo, "commit", "-q", "-m", "link")
    with pytest.raises(T.ToolError):
        T.export_source(str(repo), "HEAD", str(tmp_path / "e.tar.gz"))


def test_release_gates_and_local_tag(repo):
    res = dict((n, o) for n, o, _ in T.cut_release(str(repo), "v0.2.0"))
    assert res["version"] and res["tag-absent"] and res["clean-tree"] and not res["notes"] and not res["changelog"] and not res["recipes"]
    assert not dict((n, o) for n, o, _ in T.cut_release(str(repo), "0.2"))["version"]
    (repo / "releases" / "v0.2.0").mkdir(parents=True)
    (repo / "releases" / "v0.2.0" / "NOTES.md").write_text("notes\n")
    (repo / "CHANGELOG.md").write_text("# Changelog\n\n## v0.2.0\n- things\n")
    # one sealed recipe so that the recipe gate has something to verify
    import shutil
    src = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "runtimes", "dense")
    shutil.copytree(src, repo / "runtimes" / "dense")
    git(repo, "add", "-A")
    git(repo, "commit", "-q", "-m", "release files")
    out = io.StringIO()
    assert T.main(["cut-release", "--version", "v0.2.0", "--repo", str(repo), "--tag"], out=out) == 0, out.getvalue()
    assert "PASS tag-created" in out.getvalue()
    assert not dict((n, o) for n, o, _ in T.cut_release(str(repo), "v0.2.0"))["tag-absent"]
