import json
import os
import shutil

import pytest

from rexl3_b200.recipes import RecipeError, resolve

ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "runtimes")
SITE = {"model_dir": "/models/dense-27b", "http_port": 8123, "http_host": "0.0.0.0"}


def test_shipped_recipe_resolves_to_known_flags():
    r = resolve(ROOT, "dense", "dense-27b", SITE)
    assert r.version == "v1" and r.profile == "b200-single-64x8k"
    assert r.argv[:2] == ["--model", "/models/dense-27b"] and "8123" in r.argv and r.http_port == 8123
    from rexl3_b200.server.main import parser
    parser().parse_args(r.argv)                                     # the rendered argv is a valid command line of the serving binary
    tp = resolve(ROOT, "dense", "dense-27b", SITE, profile="b200-tp8-long-context")
    assert tp.env["NCCL_NVLS_ENABLE"] == "0"


def test_refusals(tmp_path):
    dst = tmp_path / "runtimes"
    shutil.copytree(ROOT, dst)
    with pytest.raises(RecipeError, match="site file lacks"):
        resolve(str(dst), "dense", "dense-27b", {"http_port": 1})
    p = dst / "dense" / "dense-27b" / "v1" / "profile.json"
    doc = json.loads(p.read_text())
    doc["profiles"]["b200-single-64x8k"]["argv"] += ["--no-such-flag"]
    p.write_text(json.dumps(doc))
    with pytest.raises(RecipeError, match="does not know"):
        resolve(str(dst), "dense", "dense-27b", SITE)
    doc["profiles"]["b200-single-64x8k"]["argv"][-1] = "@DRAFT_DIR@"
    p.write_text(json.dumps(doc))
    with pytest.raises(RecipeError, match="unrendered placeholder"):
        resolve(str(dst), "dense", "dense-27b", SITE)
    doc["state"] = "draft"
    p.write_text(json.dumps(doc))
    with pytest.raises(RecipeError, match="not 'final'"):
        resolve(str(dst), "dense", "dense-27b", SITE)
    with pytest.raises(RecipeError):
        resolve(str(dst), "dense", "nope", SITE)


def test_sealed_tree_verification(tmp_path):
    from rexl3_b200.recipes import seal, verify_tree
    assert verify_tree(os.path.join(ROOT, "dense", "dense-27b", "v1")) == []          # the shipped tree is sealed and intact
    dst = tmp_path / "v1"
    shutil.copytree(os.path.join(ROOT, "dense", "dense-27b", "v1"), dst)
    (dst / "launch.sh").write_text("#!/bin/sh\necho changed\n")
    (dst / "extra.txt").write_text("x")
    os.remove(dst / "profile.json")
    probs = verify_tree(str(dst))
    assert "changed: launch.sh" in probs and "unlisted: extra.txt" in probs and "missing: profile.json" in probs
    (dst / "profile.json").write_text("{}")
    seal(str(dst))
    assert verify_tree(str(dst)) == []
