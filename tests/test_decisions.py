"""/v1/decisions: the scoring math, strict validation, and the route end to end over the CPU dense backend."""
import math

import numpy as np
import pytest

from rexl3_b200.server import decisions as dec
from rexl3_b200.server.api import ApiError
from rexl3_b200.server.text import ChatFormat
from rexl3_b200.server.tokenizer import ByteTokenizer


def test_math_full_row_logsumexp_and_label_conditioned_probabilities():
    row = np.array([0.0, 1.0, 2.0, -50.0, 3.0], dtype=np.float32)
    want = math.log(sum(math.exp(float(v)) for v in row))
    assert abs(dec.logsumexp_full_row(row) - want) < 1e-12
    p = dec.Prepared("q", "score", ["0", "1", "2"], ["0", "1", "2"], "", [1], [0, 1, 2])
    a = dec.score_question(p, row, 0.5)
    e = [math.exp((v - 2.0) / 0.5) for v in (0.0, 1.0, 2.0)]
    assert abs(a["probabilities"]["2"] - e[2] / sum(e)) < 1e-12 and abs(sum(a["probabilities"].values()) - 1) < 1e-12
    assert abs(a["score"] - sum(i * x / sum(e) for i, x in enumerate(e))) < 1e-12 and a["choice"] == "2"
    assert abs(a["logprobs"]["0"] - (0.0 - want)) < 1e-12
    assert abs(a["label_mass"] - sum(math.exp(float(v) - want) for v in row[:3])) < 1e-12
    tie = dec.score_question(dec.Prepared("q", "yes_no", ["yes", "no"], ["y", "n"], "", [1], [0, 0]), row, 1.0)
    assert tie["answer"] == "yes"                    # first index wins ties


def test_validation_is_strict():
    tok, fmt = ByteTokenizer(512), ChatFormat()
    ok = {"input": "text", "questions": [{"id": "a", "type": "yes_no", "question": "good?", "yes": "y", "no": "n"}]}
    prepared, temp, echo = dec.prepare(ok, tok, fmt, 4096)
    assert prepared[0].label_ids == [ord("y"), ord("n")] and temp == 1.0 and not echo
    for bad in ({**ok, "extra": 1}, {**ok, "temperature": 0}, {**ok, "questions": []}, {"input": "", "questions": ok["questions"]},
                {**ok, "questions": [{"id": "a", "type": "choice", "question": "q", "options": ["only one"]}]},
                {**ok, "questions": [{"id": "a", "type": "yes_no", "question": "q", "yes": "yes", "no": "n"}]},      # "yes" is three byte tokens
                {**ok, "questions": [{"id": "a", "type": "score", "question": "q", "levels": 11}]},
                {**ok, "questions": ok["questions"] * 2}, {**ok, "prompt_format_version": 2}):
        with pytest.raises(ApiError):
            dec.prepare(bad, tok, fmt, 4096)
    with pytest.raises(ApiError) as e:
        dec.prepare(ok, tok, fmt, 8)
    assert e.value.code == "context_length_exceeded"


@pytest.mark.timeout(120)
def test_route_scores_with_the_cpu_backend():
    from starlette.testclient import TestClient
    from rexl3_b200.server.main import make_app, parser
    args = parser().parse_args(["--backend", "cpu", "--random-init", "tiny-llama", "--slots", "2", "--max-model-len", "512", "--prefill-chunk", "64"])
    app, handle = make_app(args)
    assert handle.wait_ready(60)
    try:
        with TestClient(app) as c:
            body = {"input": "The sky is blue.", "temperature": 0.7, "return_prompt_token_ids": True,
                    "questions": [{"id": "c", "type": "choice", "question": "Colour?", "options": ["blue", {"name": "red", "description": "warm"}]},
                                  {"id": "s", "type": "score", "question": "How sure?", "levels": 3}]}
            r = c.post("/v1/decisions", json=body)
            assert r.status_code == 200, r.text
            doc = r.json()
            assert doc["object"] == "decision" and doc["usage"]["completion_tokens"] == 0
            a = doc["answers"]["c"]
            assert set(a["probabilities"]) == {"blue", "red"} and abs(sum(a["probabilities"].values()) - 1) < 1e-9 and a["choice"] in ("blue", "red")
            assert 0 < a["label_mass"] < 1 and isinstance(a["prompt_token_ids"], list)
            assert 0 <= doc["answers"]["s"]["score"] <= 2
            again = c.post("/v1/decisions", json=body).json()
            assert again["answers"] == doc["answers"]              # scoring leaves nothing behind in the slot
            assert c.post("/v1/decisions", json={**body, "nope": 1}).status_code == 400
    finally:
        handle.stop()
