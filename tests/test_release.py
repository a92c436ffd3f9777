"""Release governance over recipe trees: verify-all on the shipped trees, promotion rules, evidence document."""
import json
import os
import shutil

import pytest

from rexl3_b200 import recipes, release

ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "runtimes")


def test_shipped_trees_are_intact_resolvable_and_approved():
    assert release.verify_all(ROOT) == []
    fams = {(f, m) for f, m, _ in release._trees(ROOT)}
    assert {("dense", "dense-27b"), ("hybrid", "gdn-hybrid-27b"), ("hybrid", "hybrid-h-56l"), ("moe", "moe-spec-30b")} <= fams


def _copy(tmp_path):
    root = str(tmp_path / "runtimes")
    shutil.copytree(ROOT, root)
    return root


def test_promotion_needs_a_sealed_final_approved_version(tmp_path):
    root = _copy(tmp_path)
    mdir = os.path.join(root, "dense", "dense-27b")
    v2 = os.path.join(mdir, "v2")
    shutil.copytree(os.path.join(mdir, "v1"), v2)
    os.remove(os.path.join(v2, "approval.json"))
    recipes.seal(v2)
    with pytest.raises(recipes.RecipeError, match="approval"):
        release.promote(root, "dense", "dense-27b", "v2")
    json.dump({"approved": True, "approved_by": "someone"}, open(os.path.join(v2, "approval.json"), "w"))
    with pytest.raises(recipes.RecipeError, match="manifest"):           # the approval was added after sealing
        release.promote(root, "dense", "dense-27b", "v2")
    recipes.seal(v2)
    prof = json.load(open(os.path.join(v2, "profile.json")))
    prof["state"] = "draft"
    json.dump(prof, open(os.path.join(v2, "profile.json"), "w"))
    recipes.seal(v2)
    with pytest.raises(recipes.RecipeError, match="final"):
        release.promote(root, "dense", "dense-27b", "v2")
    prof["state"] = "final"
    json.dump(prof, open(os.path.join(v2, "profile.json"), "w"))
    recipes.seal(v2)
    assert release.promote(root, "dense", "dense-27b", "v2") == "v2"
    assert open(os.path.join(mdir, "LATEST")).read().strip() == "v2"
    assert release.verify_all(root) == []
    assert release.main(["promote", "--root", root, "--family", "dense", "--model", "dense-27b", "--version", "v9"]) == 2


def test_verify_all_reports_damage_and_evidence_lists_recipes(tmp_path):
    root = _copy(tmp_path)
    with open(os.path.join(root, "moe", "moe-spec-30b", "v1", "launch.sh"), "a") as f:
        f.write("# edited after sealing\n")
    open(os.path.join(root, "hybrid", "hybrid-h-56l", "LATEST"), "w").write("v7\n")
    bad = release.verify_all(root)
    assert any("moe/moe-spec-30b/v1: changed: launch.sh" in b for b in bad) and any("LATEST names 'v7'" in b for b in bad)
    doc = release.evidence(root, str(tmp_path))
    assert doc["schema"] == "rexl3.release-evidence.v1" and doc["problems"] == bad
    dense = next(r for r in doc["recipes"] if r["model"] == "dense-27b")
    assert dense["version"] == "v1" and len(dense["manifest_sha256"]) == 64 and dense["approval"]["approved_by"]
