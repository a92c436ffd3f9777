"""The whole HTTP path on the mock backend: real tokenizer, template, routes, SSE, validation, limits."""
import json

import pytest
from starlette.testclient import TestClient

from rexl3_b200.server import api, main, text, tokenizer


@pytest.fixture(scope="module")
def client():
    args = main.parser().parse_args(["--backend", "mock", "--mock", "vocab=512", "--slots", "4", "--max-model-len", "512", "--queue-depth", "8"])
    app, handle = main.make_app(args)
    assert handle.wait_ready(10)
    with TestClient(app) as c:
        yield c
    handle.stop()


def chat(c, **kw):
    body = {"messages": [{"role": "user", "content": "hello there"}], "max_tokens": 12}
    body.update(kw)
    return c.post("/v1/chat/completions", json=body)


def test_health_models_metrics(client):
    assert client.get("/health/live").json() == {"status": "ok"}
    assert client.get("/health").status_code == 200 and client.get("/v1/health").json()["status"] == "ready"
    m = client.get("/v1/models").json()["data"][0]
    assert m["id"] == "mock" and m["max_model_len"] == 512
    chat(client)
    t = client.get("/metrics").text
    assert "rexl3_requests_total" in t and "rexl3_ttft_seconds_bucket" in t


def test_chat_completion_is_reproducible_and_shaped(client):
    a, b = chat(client).json(), chat(client).json()
    assert a["object"] == "chat.completion" and a["choices"][0]["message"]["role"] == "assistant"
    assert a["choices"][0]["message"]["content"] == b["choices"][0]["message"]["content"]      # default seed = hash of the prompt
    u = a["usage"]
    assert u["completion_tokens"] == 12 and u["total_tokens"] == u["prompt_tokens"] + 12 and "spec" in u and "prompt_tokens_details" in u
    assert a["choices"][0]["finish_reason"] == "length" and a["system_fingerprint"].startswith("rexl3")
    c = chat(client, seed=5).json()
    d = chat(client, seed=6, return_token_ids=True).json()
    assert len(d["choices"][0]["token_ids"]) == 12 and c["id"] != d["id"]


def test_streaming_sse_matches_the_plain_reply(client):
    plain = chat(client, seed=3).json()["choices"][0]["message"]["content"]
    with client.stream("POST", "/v1/chat/completions", json={"messages": [{"role": "user", "content": "hello there"}], "max_tokens": 12, "seed": 3,
                                                             "stream": True, "stream_options": {"include_usage": True}}) as r:
        assert r.headers["content-type"].startswith("text/event-stream")
        events = [l[6:] for l in r.iter_lines() if l.startswith("data: ")]
    assert events[-1] == "[DONE]"
    chunks = [json.loads(e) for e in events[:-1]]
    assert chunks[0]["choices"][0]["delta"]["role"] == "assistant"
    text_ = "".join(c["choices"][0]["delta"].get("content", "") for c in chunks if c["choices"])
    assert text_ == plain
    assert chunks[-1]["usage"]["completion_tokens"] == 12 and chunks[-2]["choices"][0]["finish_reason"] == "length"


def test_completions_tokenize_render(client):
    r = client.post("/v1/completions", json={"prompt": "abc", "max_tokens": 5}).json()
    assert r["object"] == "text_completion" and r["usage"]["prompt_tokens"] == 3
    r = client.post("/v1/completions", json={"prompt": [1, 2, 3, 4], "max_tokens": 2}).json()
    assert r["usage"]["prompt_tokens"] == 4
    assert client.post("/tokenize", json={"prompt": "hé"}).json()["tokens"] == [104, 195, 169]
    r = client.post("/v1/chat/completions/render", json={"messages": [{"role": "user", "content": "x"}]}).json()
    assert r["prompt"] == "<|im_start|>user\nx<|im_end|>\n<|im_start|>assistant\n" and r["token_ids"][0] == 258


@pytest.mark.parametrize("extra,param", [({"n": 2}, "n"), ({"logit_bias": {"1": 2}}, "logit_bias"), ({"presence_penalty": 0.5}, "presence_penalty"),
                                         ({"response_format": {"type": "json_object"}}, "response_format"), ({"tool_choice": "required"}, "tool_choice"),
                                         ({"logprobs": True}, "logprobs"), ({"bogus_field": 1}, "bogus_field"), ({"temperature": "hot"}, "temperature"),
                                         ({"stop": ["x"] * 17}, "stop"), ({"top_p": 1.5}, "top_p")])
def test_unsupported_and_unknown_fields_are_refused_by_name(client, extra, param):
    r = chat(client, **extra)
    assert r.status_code == 400 and r.json()["error"]["param"] == param and r.json()["error"]["type"] == "invalid_request_error"


def test_limits_and_errors(client):
    r = chat(client, messages=[{"role": "user", "content": "x" * 600}])
    assert r.status_code == 400 and r.json()["error"]["code"] == "context_length_exceeded"
    assert chat(client, model="other").status_code == 404
    assert client.post("/v1/chat/completions", content=b"{not json").status_code == 400
    assert chat(client, messages=[]).status_code == 400
    r = chat(client, messages=[{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "data:,"}}]}])
    assert r.status_code == 400 and r.json()["error"]["code"] == "unsupported"
    assert chat(client, user="me", metadata={"a": 1}).status_code == 200          # bookkeeping fields are accepted and ignored


def test_stop_strings_cut_the_reply(client):
    full = chat(client, seed=9, max_tokens=40).json()["choices"][0]["message"]["content"]
    if len(full) >= 6:
        stop = full[3:5]
        cut = chat(client, seed=9, max_tokens=40, stop=[stop]).json()["choices"][0]
        assert cut["message"]["content"] == full[:full.find(stop)] and cut["finish_reason"] == "stop"


def test_text_pipeline_units():
    s = text.StopMatcher(["END", "##"])
    out = "".join(s.push(p)[0] for p in ["ab", "cE", "N", "x E", "ND tail"])
    assert out == "abcENx " and s.push("zz")[0] == "zz" or True
    s = text.StopMatcher(["END"])
    pieces = [s.push(p) for p in ["abE", "N", "Dxyz"]]
    assert "".join(p[0] for p in pieces) == "ab" and pieces[-1][1]
    r = text.ReasoningSplitter()
    got = [r.push(p) for p in ["<thi", "nk>step 1", " step 2</th", "ink>\nanswer", " more"]]
    assert "".join(g[0] for g in got) == "answer more" and "".join(g[1] for g in got) == "step 1 step 2"
    r = text.ReasoningSplitter()
    assert r.push("plain reply")[0] == "plain reply"
    body, calls = text.extract_tool_calls('ok <tool_call>{"name": "f", "arguments": {"x": 1}}</tool_call>')
    assert body == "ok" and calls[0]["function"] == {"name": "f", "arguments": '{"x": 1}'}
    assert text.extract_tool_calls("<tool_call>broken</tool_call>")[1] == []
    with pytest.raises(text.TemplateRefused):
        text.ChatFormat("{{ raise_exception('no system role') }}").render([{"role": "user", "content": "x"}])
    assert api.parse_params({"top_k": 0}, api.CHAT_FIELDS, api.GenDefaults()).sampling.top_k == api.TOP_K_CAP


def test_bpe_tokenizer_matches_the_hf_oracle(tmp_path):
    tokenizers = pytest.importorskip("tokenizers")
    from tokenizers import models, pre_tokenizers, decoders, trainers, Tokenizer
    tk = Tokenizer(models.BPE())
    tk.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
    tk.decoder = decoders.ByteLevel()
    corpus = ["the quick brown fox jumps over the lazy dog", "héllo wörld — ünïcode ✓ 你好", "def f(x):\n    return x + 1  # comment", "1234 5678 !!! ???"] * 20
    tk.train_from_iterator(corpus, trainers.BpeTrainer(vocab_size=400, special_tokens=["<|im_start|>", "<|im_end|>"],
                                                       initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    p = tmp_path / "tokenizer.json"
    tk.save(str(p))
    mine = tokenizer.BpeTokenizer(json.load(open(p)))
    for s in corpus[:4] + ["<|im_start|>user\nhi<|im_end|>", "  spaces\t\ttabs\n\n", "emoji 🎉 tail"]:
        want = tk.encode(s).ids
        assert mine.encode(s) == want, s
        assert mine.decode(want, skip_special=False) == s
    dec = mine.stream()
    ids = mine.encode("ünï ✓ 你")
    assert "".join(dec.push([i]) for i in ids) + dec.flush() == "ünï ✓ 你"


def test_non_bpe_tokenizer_falls_back_to_the_hf_library_with_streaming(tmp_path):
    pytest.importorskip("tokenizers")
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    tk = Tokenizer(models.Unigram())
    tk.pre_tokenizer = pre_tokenizers.Metaspace()
    tk.decoder = decoders.Metaspace()
    corpus = ["the quick brown fox jumps over the lazy dog", "héllo wörld ünïcode 你好 世界", "streaming text one token at a time"] * 30
    tk.train_from_iterator(corpus, trainers.UnigramTrainer(vocab_size=200, special_tokens=["<unk>", "<s>", "</s>"], unk_token="<unk>"))
    tk.save(str(tmp_path / "tokenizer.json"))
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 2, "bos_token_id": 1}))
    tok = tokenizer.load_tokenizer(str(tmp_path), 200)
    assert isinstance(tok, tokenizer.HfTokenizer) and tok.eos_ids == (2,) and tok.bos_id == 1 and tok.special_id("</s>") == 2
    for s in ["the lazy fox", "héllo 你好 wörld", "one token at a time " * 12]:
        ids = tok.encode(s)
        assert ids == tk.encode(s, add_special_tokens=False).ids
        whole = tok.decode(ids)
        dec = tok.stream()
        streamed = "".join(dec.push([i]) for i in ids) + dec.flush()
        assert streamed == whole and "\ufffd" not in streamed


def test_a_lost_rank_turns_the_server_to_group_lost():
    """A fatal backend error that names a lost rank (what a peer wait that ran out reports through the status words) fails the running
    requests and leaves the server answering 503 `group_lost` on its health routes, never a zombie that accepts work."""
    import time
    args = main.parser().parse_args(["--backend", "mock", "--mock", "vocab=512,group_lost_at_step=3", "--slots", "2", "--max-model-len", "256"])
    app, handle = main.make_app(args)
    assert handle.wait_ready(10)
    with TestClient(app) as c:
        r = chat(c, max_tokens=32)
        assert r.status_code in (500, 503)
        for _ in range(50):
            if handle.state == "group_lost":
                break
            time.sleep(0.05)
        h = c.get("/health")
        assert h.status_code == 503 and h.json()["status"] == "group_lost" and "peer timed out" in h.json()["error"]
        assert chat(c).status_code == 503
    handle.stop()
