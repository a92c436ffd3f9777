"""The memory plan tool over every family."""
import json

from rexl3_b200 import plan


def test_plan_numbers_are_consistent_across_families():
    d = plan.plan(plan.find_config("dense-27b"), slots=64, max_model_len=8704)
    assert d["family"] == "dense_gqa" and d["kv_bytes_per_token"] == 2 * 8 * 128 * 2 * 64 and d["fits"]
    assert 11e9 < d["weight_bytes"] < 14e9
    f8 = plan.plan(plan.find_config("dense-27b"), slots=64, max_model_len=8704, kv_dtype="fp8")
    assert f8["kv_bytes_per_token"] * 2 == d["kv_bytes_per_token"] and f8["kv_tokens_that_fit"] > 1.9 * d["kv_tokens_that_fit"]
    one = plan.plan(plan.find_config("mla-moe-671b"), gpus=1)
    eight = plan.plan(plan.find_config("mla-moe-671b"), gpus=8, slots=64, max_model_len=8704)
    assert not one["fits"] and eight["fits"] and eight["per_gpu"]["weights"] * 8 <= one["weight_bytes"]
    h = plan.plan(plan.find_config("gdn-hybrid-27b"), slots=16, max_model_len=8704)
    assert h["family"] == "hybrid" and h["per_gpu"]["recurrent_state"] == 16 * h["state_bytes_per_slot"] > 0
    assert h["kv_bytes_per_token"] == 2 * 8 * 128 * 2 * 16           # only the 16 attention layers cache keys and values
    assert plan.plan(plan.find_config("moe-spec-30b"))["family"] == "moe_gqa"


def test_cli(capsys, tmp_path):
    assert plan.main(["--config", "tiny-llama", "--slots", "4", "--max-model-len", "512"]) == 0
    assert json.loads(capsys.readouterr().out)["fits"] is True
    assert plan.main(["--config", "no-such-model"]) == 2
    assert plan.main(["--config", "mla-moe-671b"]) == 1
