"""Chat-format registry, tool syntaxes with schema typing, reasoning controls and request budgets (all host-side)."""
import json
import threading
import time

import pytest

from rexl3_b200.server import budget, formats as F


def test_registry_finds_families_and_refuses_unknown_ones_by_listing_what_exists():
    assert F.find({"architectures": ["Qwen3_5ForCausalLM"]}) is F.QwenFormat
    assert F.find({"model_type": "glm5_next"}) is F.GlmFormat
    assert F.find({"model_type": "rexl3_dense"}) is F.FamilyFormat
    assert F.find({"model_type": "whatever"}, override="deepseek_v41") is F.DeepseekV41Format
    with pytest.raises(F.FormatRefused) as e:
        F.find({"architectures": ["SomethingElseForCausalLM"]})
    assert "qwen" in str(e.value) and "bailing_moe_v3" in str(e.value) and "--chat-format" in str(e.value)
    with pytest.raises(F.FormatRefused):
        F.find({}, override="nope")
    assert set(F.registered()) == {"chatml", "qwen", "glm5_next", "mimo", "nemotron_omni", "minicpmv", "deepseek_v41", "bailing_moe_v3"}


def test_open_format_binds_the_folder_template_and_tokens(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps({"architectures": ["Qwen3_5ForCausalLM"]}))
    (tmp_path / "chat_template.jinja").write_text("{{ bos_token }}{% for m in messages %}[{{ m['role'] }}]{{ m['content'] }}{% endfor %}<think>\n")
    (tmp_path / "tokenizer_config.json").write_text(json.dumps({"bos_token": {"content": "<s>"}, "eos_token": "</s>"}))
    f = F.open_format(str(tmp_path))
    text = f.render([{"role": "user", "content": "hi"}])
    assert f.id == "qwen" and text == "<s>[user]hi<think>" and f.starts_in_reasoning(text)     # jinja drops one trailing newline, as HF does
    (tmp_path / "chat_template.jinja").write_text("{% for %}")
    with pytest.raises(F.FormatRefused):
        F.open_format(str(tmp_path))


TOOLS = [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object", "properties": {
    "city": {"type": "string"}, "days": {"type": "integer"}, "metric": {"type": "boolean"}, "tags": {"type": "array"},
    "unit": {"$ref": "#/$defs/Unit"}, "zip": {"anyOf": [{"type": "integer"}, {"type": "string"}]}},
    "$defs": {"Unit": {"enum": ["c", "f"]}}}}}]


def test_function_block_calls_are_typed_from_the_schema():
    text = ("Let me check.\n<tool_call>\n<function=get_weather>\n<parameter=city>\n42\n</parameter>\n<parameter=days>\n3\n</parameter>\n"
            "<parameter=metric>\ntrue\n</parameter>\n<parameter=tags>\n[\"a\", 1]\n</parameter>\n<parameter=unit>\nc\n</parameter>\n"
            "<parameter=zip>\n0123x\n</parameter>\n<parameter=extra>\n{\"k\": 1}\n</parameter>\n</function>\n</tool_call>")
    visible, calls = F.QwenFormat().split_tools(text, TOOLS)
    assert visible == "Let me check." and len(calls) == 1 and calls[0]["function"]["name"] == "get_weather"
    args = json.loads(calls[0]["function"]["arguments"])
    # a string parameter keeps "42" as text; the integer, boolean and array are read; the union falls back to the string; undeclared -> JSON
    assert args == {"city": "42", "days": 3, "metric": True, "tags": ["a", 1], "unit": "c", "zip": "0123x", "extra": {"k": 1}}
    # malformed blocks stay in the text, nothing runs with half its arguments
    bad = "<tool_call>\n<function=get_weather>\n<parameter=city>\nx\n</function>\n</tool_call>"
    visible, calls = F.QwenFormat().split_tools(bad, TOOLS)
    assert calls == [] and visible == bad
    assert F.QwenFormat().split_tools(text, TOOLS, tool_choice="none") == (text, [])


def test_arg_pair_json_dsml_and_list_syntaxes():
    glm = "<tool_call>get_weather<arg_key>city</arg_key><arg_value>Paris</arg_value>\n<arg_key>days</arg_key>\n<arg_value>2</arg_value></tool_call><tool_call>get_time</tool_call>"
    _, calls = F.GlmFormat().split_tools(glm, TOOLS + [{"type": "function", "function": {"name": "get_time"}}])
    assert [c["function"]["name"] for c in calls] == ["get_weather", "get_time"]
    assert json.loads(calls[0]["function"]["arguments"]) == {"city": "Paris", "days": 2} and json.loads(calls[1]["function"]["arguments"]) == {}
    assert F.GlmFormat().split_tools("<tool_call>bad name<arg_key>k</arg_key><arg_value>v</arg_value></tool_call>", TOOLS)[1] == []
    _, calls = F.FamilyFormat().split_tools('ok <tool_call>{"name": "get_weather", "arguments": {"city": "Rome"}}</tool_call>', TOOLS)
    assert json.loads(calls[0]["function"]["arguments"]) == {"city": "Rome"}
    d = "｜DSML｜"
    dsml = (f'<{d} calls><{d} invoke name="GET_WEATHER"><{d} parameter name="city" string="true">Oslo</{d} parameter>'
            f'<{d} parameter name="days" string="false">5</{d} parameter></{d} invoke></{d} calls>')
    _, calls = F.DeepseekV41Format().split_tools(dsml, TOOLS)
    assert calls[0]["function"]["name"] == "get_weather" and json.loads(calls[0]["function"]["arguments"]) == {"city": "Oslo", "days": 5}
    _, calls = F.NemotronOmniFormat().split_tools('<TOOLCALL>[{"name": "get_weather", "arguments": {"city": "Bonn"}}]</TOOLCALL>', TOOLS)
    assert json.loads(calls[0]["function"]["arguments"]) == {"city": "Bonn"}


def test_history_with_string_arguments_becomes_renderable():
    msgs = [{"role": "assistant", "content": "", "tool_calls": [{"type": "function", "function": {"name": "f", "arguments": "{\"a\": 1}"}}]}]
    assert F.normalize_history(msgs)[0]["tool_calls"][0]["function"]["arguments"] == {"a": 1}
    assert msgs[0]["tool_calls"][0]["function"]["arguments"] == "{\"a\": 1}"


def test_reasoning_controls_follow_the_declared_capabilities():
    q = F.QwenFormat().caps
    assert F.apply_reasoning_controls(q, {}, default_thinking="off") == ({"enable_thinking": False}, None)
    assert F.apply_reasoning_controls(q, {}, default_thinking="template") == ({}, None)
    assert F.apply_reasoning_controls(q, {"enable_thinking": True}, default_thinking="off")[0] == {"enable_thinking": True}
    assert F.apply_reasoning_controls(q, {}, thinking=True)[0] == {"enable_thinking": True}
    with pytest.raises(F.ControlRefused) as e:
        F.apply_reasoning_controls(q, {"bogus": 1})
    assert "enable_thinking" in str(e.value) and e.value.param == "chat_template_kwargs"
    with pytest.raises(F.ControlRefused):
        F.apply_reasoning_controls(q, {"enable_thinking": "yes"})
    with pytest.raises(F.ControlRefused):
        F.apply_reasoning_controls(q, {"enable_thinking": False}, thinking=True)
    with pytest.raises(F.ControlRefused):
        F.apply_reasoning_controls(q, {}, effort="high")            # this family declares no levels
    d = F.DeepseekV41Format().caps
    assert F.apply_reasoning_controls(d, {}, effort="high")[0] == {"reasoning_effort": "high", "thinking": True}
    assert F.apply_reasoning_controls(d, {}, effort="none")[0] == {"thinking": False}
    assert F.apply_reasoning_controls(d, {}, default_effort="low")[0] == {"reasoning_effort": "low", "thinking": True}
    assert F.apply_reasoning_controls(d, {"thinking": False}, default_effort="low")[0] == {"thinking": False}    # the client's own choice wins
    with pytest.raises(F.ControlRefused):
        F.apply_reasoning_controls(d, {"reasoning_effort": "low"}, effort="high")
    with pytest.raises(F.ControlRefused):
        F.apply_reasoning_controls(d, {"thinking": False}, effort="high")
    n = F.NemotronOmniFormat().caps
    kw, note = F.apply_reasoning_controls(n, {"enable_thinking": False})
    assert kw == {"enable_thinking": False} and "always opens" in note
    assert F.apply_reasoning_controls(n, {}, default_thinking="off") == ({}, None)      # a switch that cannot close the block is not inserted
    assert F.DeepseekV41Format().render([{"role": "user", "content": "x"}], thinking=True).endswith("<think>")
    assert F.BailingFormat().render([{"role": "user", "content": "x"}]).endswith("<role>ASSISTANT</role>")


def test_media_parts_are_refused_by_name_and_role_stops_are_single_tokens():
    msgs = [{"role": "user", "content": [{"type": "text", "text": "hi"}, {"type": "image_url", "image_url": {"url": "x"}}]}]
    assert "image_url" in F.QwenFormat().check_media(msgs) and F.QwenFormat().check_media([{"role": "user", "content": "x"}]) is None

    class Tok:
        def encode(self, t):
            return [7] if t == "<|im_start|>" else [1, 2]
    assert F.QwenFormat().reply_role_stops(Tok()) == [7] and F.GlmFormat().reply_role_stops(Tok()) == []


def test_limits_derive_from_the_window_and_validate():
    lim = budget.Limits.for_window(262_144)
    assert lim.rendered_bytes == 4 << 20 and lim.processing_reserve_bytes == 2 << 30
    assert budget.Limits.for_window(1024).rendered_bytes == 1 << 20
    big = budget.Limits.for_window(1 << 20)
    assert big.processing_reserve_bytes == big.tokenizer_price() > 2 << 30
    lim.processing_reserve_bytes = 1 << 20
    with pytest.raises(ValueError):
        lim.validate()
    with pytest.raises(ValueError):
        budget.Limits(json_depth=200).validate()


def test_json_node_and_depth_caps_are_iterative():
    lim = budget.Limits(json_nodes=50, json_depth=10)
    assert budget.check_json({"a": [1, 2, {"b": None}]}, lim) == 8
    with pytest.raises(budget.BudgetRefused) as e:
        budget.check_json(list(range(100)), lim)
    assert e.value.status == 413 and e.value.code == "json_too_large"
    deep = cur = []
    for _ in range(5000):           # far deeper than the interpreter's recursion limit
        nxt = []
        cur.append(nxt)
        cur = nxt
    with pytest.raises(budget.BudgetRefused) as e:
        budget.check_json(deep, budget.Limits(json_depth=100))
    assert e.value.code == "json_too_deep"
    with pytest.raises(budget.BudgetRefused):
        budget.check_rendered("x" * 2000, budget.Limits(rendered_bytes=1000))


def test_tokenizer_gate_prices_waits_in_order_and_refuses():
    g = budget.TokenizerGate(capacity=budget.TokenizerGate.price(1000), wait_s=0.3)
    with pytest.raises(budget.BudgetRefused) as e:
        g.charge(1001)
    assert e.value.status == 413
    a = g.charge(700)
    order = []

    def take(n, tag):
        try:
            with g.charge(n):
                order.append(tag)
        except budget.BudgetRefused as ex:
            order.append((tag, ex.status))
    t1 = threading.Thread(target=take, args=(600, "big"))
    t1.start()
    time.sleep(0.05)
    t2 = threading.Thread(target=take, args=(100, "small"))       # would fit now, but must not overtake the big one
    t2.start()
    time.sleep(0.05)
    assert order == [] and g.in_use() == budget.TokenizerGate.price(700)
    a.release()
    t1.join(); t2.join()
    assert order == ["big", "small"] and g.in_use() == 0 and g.waited == 2
    b = g.charge(900)
    t0 = time.monotonic()
    with pytest.raises(budget.BudgetRefused) as e:
        g.charge(500)
    assert e.value.status == 429 and 0.25 < time.monotonic() - t0 < 2.0
    b.release()
    pg = budget.PreparationGate(1, 0)
    with pg:
        with pytest.raises(budget.BudgetRefused) as e:
            with pg:
                pass
        assert e.value.status == 429


@pytest.fixture(scope="module")
def qwen_client():
    from starlette.testclient import TestClient
    from rexl3_b200.server import main
    args = main.parser().parse_args(["--backend", "mock", "--mock", "vocab=512", "--slots", "4", "--max-model-len", "512", "--queue-depth", "8",
                                     "--chat-format", "qwen", "--max-json-nodes", "200", "--max-rendered-prompt-mib", "0.001"])
    app, handle = main.make_app(args)
    assert handle.wait_ready(10)
    with TestClient(app) as c:
        yield c
    handle.stop()


def test_http_applies_family_controls_budgets_and_exposes_capabilities(qwen_client):
    c = qwen_client
    m = c.get("/v1/models").json()["data"][0]
    assert m["chat_format"] == "qwen" and m["reasoning"]["thinking_switch"] == "enable_thinking" and m["reasoning"]["template_thinks_by_default"]
    msgs = [{"role": "user", "content": "x"}]
    r = c.post("/v1/chat/completions/render", json={"messages": msgs}).json()
    assert r["prompt"].endswith("<think>\n\n</think>\n\n")                      # --default-thinking off: the switch is inserted as false
    r = c.post("/v1/chat/completions/render", json={"messages": msgs, "thinking": True}).json()
    assert r["prompt"].endswith("<think>\n")
    r = c.post("/v1/chat/completions/render", json={"messages": msgs, "chat_template_kwargs": {"bogus": 1}})
    assert r.status_code == 400 and r.json()["error"]["param"] == "chat_template_kwargs"
    r = c.post("/v1/chat/completions/render", json={"messages": msgs, "reasoning_effort": "high"})
    assert r.status_code == 400 and r.json()["error"]["param"] == "reasoning_effort"
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "u"}}]}]})
    assert r.status_code == 400 and r.json()["error"]["code"].startswith("unsupported")
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "y" * 2000}], "max_tokens": 2})
    assert r.status_code == 413 and r.json()["error"]["code"] == "prompt_too_large"
    r = c.post("/v1/chat/completions", json={"messages": msgs, "metadata": {"k": list(range(300))}})
    assert r.status_code == 413 and r.json()["error"]["code"] == "json_too_large"
    ok = c.post("/v1/chat/completions", json={"messages": msgs, "max_tokens": 4, "thinking": True})
    assert ok.status_code == 200
