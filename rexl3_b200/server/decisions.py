"""`POST /v1/decisions`: strict validation, the closed chat prompt of each question, the one-token label gate, and the label-scoring
math over a full-vocabulary logits row.  Pure: no engine, no HTTP - the route hands each prepared question to the engine's score
path and gives the rows back to `build_response`.

Math (host-side float64, compensated summation): label-conditioned probabilities p_i = softmax(label_logits / temperature) over the K
label logits only (max-shifted); per-label logprobs logit_i - logsumexp(full row) against the WHOLE vocabulary; label_mass = sum of
exp(logprob_i); `choice` picks the argmax probability (first index wins ties), `score` is sum(index * p_index) over 0-based levels,
`yes_no` adds nothing; completion_tokens is always 0.  Behaviour parity: reference crates/server/src/decisions.rs:1-17 (format v1).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

from .api import ApiError, bad

PROMPT_FORMAT_VERSION = 1
TOP_FIELDS = {"input", "questions", "temperature", "chat_template_kwargs", "prompt_format_version", "return_prompt_token_ids", "model"}
FIELDS = {"choice": {"id", "type", "question", "options"}, "score": {"id", "type", "question", "levels"}, "yes_no": {"id", "type", "question", "yes", "no"}}
MAX_OPTIONS, MAX_LEVELS, MAX_QUESTIONS, MAX_PROMPT_BYTES = 26, 10, 64, 8 << 20


@dataclass
class Prepared:
    id: str
    kind: str
    names: list            # response keys per label
    labels: list           # label spellings shown in the prompt
    prompt_text: str
    prompt: list
    label_ids: list


def _kahan(xs) -> float:
    s = c = 0.0
    for x in xs:
        y = x - c
        t = s + y
        c = (t - s) - y
        s = t
    return s


def logsumexp_full_row(row) -> float:
    peak = -math.inf
    for v in row:
        v = float(v)
        if v != v:
            return math.nan
        if v > peak:
            peak = v
    if not math.isfinite(peak):
        return peak
    return peak + math.log(_kahan(math.exp(float(v) - peak) for v in row))


def _one_token(tok, text: str, what: str) -> int:
    ids = tok.encode(text, allow_special=False)
    if len(ids) != 1:
        raise bad(f"label {text!r} of {what} is {len(ids)} tokens in the served tokenizer; labels must be single tokens", "questions", "label_not_single_token")
    return int(ids[0])


def prepare(body, tok, fmt, max_model_len: int) -> tuple:
    """-> (list[Prepared], temperature, return_prompt_token_ids)."""
    if not isinstance(body, dict):
        raise bad("the request body must be a JSON object")
    unknown = set(body) - TOP_FIELDS
    if unknown:
        raise bad(f"unknown field {sorted(unknown)[0]!r}", sorted(unknown)[0], "unknown_field")
    if body.get("prompt_format_version", PROMPT_FORMAT_VERSION) != PROMPT_FORMAT_VERSION:
        raise bad(f"prompt_format_version must be {PROMPT_FORMAT_VERSION}", "prompt_format_version")
    text = body.get("input")
    if not isinstance(text, str) or not text:
        raise bad("'input' must be a non-empty string", "input")
    if len(text.encode()) > MAX_PROMPT_BYTES:
        raise bad("'input' is too large", "input")
    temp = body.get("temperature", 1.0)
    if isinstance(temp, bool) or not isinstance(temp, (int, float)) or not math.isfinite(temp) or temp <= 0:
        raise bad("'temperature' must be a finite number > 0", "temperature")
    qs = body.get("questions")
    if not isinstance(qs, list) or not qs or len(qs) > MAX_QUESTIONS:
        raise bad(f"'questions' must be a list of 1..{MAX_QUESTIONS} questions", "questions")
    tk = body.get("chat_template_kwargs") or {}
    if not isinstance(tk, dict):
        raise bad("'chat_template_kwargs' must be an object", "chat_template_kwargs")
    out, seen = [], set()
    for q in qs:
        if not isinstance(q, dict) or q.get("type") not in FIELDS:
            raise bad("every question needs a 'type' of choice, score or yes_no", "questions")
        kind = q["type"]
        extra = set(q) - FIELDS[kind]
        if extra:
            raise bad(f"unknown field {sorted(extra)[0]!r} in a {kind} question", "questions", "unknown_field")
        qid, qt = q.get("id"), q.get("question")
        if not isinstance(qid, str) or not qid or qid in seen:
            raise bad("question ids must be distinct non-empty strings", "questions")
        seen.add(qid)
        if not isinstance(qt, str) or not qt:
            raise bad(f"question {qid!r} has no text", "questions")
        if kind == "choice":
            opts = q.get("options")
            if not isinstance(opts, list) or not 2 <= len(opts) <= MAX_OPTIONS:
                raise bad(f"question {qid!r}: 2..{MAX_OPTIONS} options", "questions")
            names, lines = [], []
            for i, o in enumerate(opts):
                if isinstance(o, str):
                    o = {"name": o}
                if not isinstance(o, dict) or set(o) - {"name", "description"} or not isinstance(o.get("name"), str) or not o["name"]:
                    raise bad(f"question {qid!r}: every option needs a 'name'", "questions")
                if o["name"] in names:
                    raise bad(f"question {qid!r}: option names must be distinct", "questions")
                names.append(o["name"])
                lines.append(f"{chr(65 + i)}. {o['name']}" + (f" - {o['description']}" if o.get("description") else ""))
            labels = [chr(65 + i) for i in range(len(opts))]
            ask = f"{qt}\n" + "\n".join(lines) + "\nAnswer with the letter only."
        elif kind == "score":
            lv = q.get("levels")
            if isinstance(lv, bool) or not isinstance(lv, int) or not 2 <= lv <= MAX_LEVELS:
                raise bad(f"question {qid!r}: 'levels' must be an integer in 2..{MAX_LEVELS}", "questions")
            labels = [str(i) for i in range(lv)]
            names = list(labels)
            ask = f"{qt}\nAnswer with one digit from 0 to {lv - 1} only."
        else:
            labels = [q.get("yes", "yes"), q.get("no", "no")]
            if not all(isinstance(x, str) and x for x in labels) or labels[0] == labels[1]:
                raise bad(f"question {qid!r}: 'yes' and 'no' must be distinct non-empty strings", "questions")
            names = ["yes", "no"]
            ask = f"{qt}\nAnswer with {labels[0]} or {labels[1]} only."
        prompt_text = fmt.render([{"role": "user", "content": f"{text}\n\n{ask}"}], add_generation_prompt=True, **{"enable_thinking": False, **tk})
        ids = tok.encode(prompt_text, allow_special=True)
        if len(ids) + 1 > max_model_len:
            raise ApiError(400, f"question {qid!r}: the prompt is {len(ids)} tokens, the context window holds {max_model_len}", code="context_length_exceeded")
        out.append(Prepared(qid, kind, names, labels, prompt_text, [int(t) for t in ids], [_one_token(tok, lb, f"question {qid!r}") for lb in labels]))
    return out, float(temp), bool(body.get("return_prompt_token_ids", False))


def score_question(p: Prepared, row, temperature: float) -> dict:
    n = len(row)
    if any(not 0 <= i < n for i in p.label_ids):
        raise ApiError(500, "a label id is outside the logits row", "server_error")
    lse = logsumexp_full_row(row)
    ll = [float(row[i]) for i in p.label_ids]
    if lse != lse or any(v != v for v in ll):
        raise ApiError(500, "the model returned a NaN logit", "server_error")
    peak = max(ll)
    ex = [math.exp((v - peak) / temperature) for v in ll]
    z = _kahan(ex)
    probs = [e / z for e in ex]
    logprobs = [v - lse for v in ll]
    ans = {"type": p.kind, "probabilities": dict(zip(p.names, probs)), "logprobs": dict(zip(p.names, logprobs)),
           "label_mass": _kahan(math.exp(v) for v in logprobs)}
    best = max(range(len(probs)), key=lambda i: (probs[i], -i))
    if p.kind == "choice":
        ans["choice"] = p.names[best]
    elif p.kind == "score":
        ans["score"] = _kahan(i * pr for i, pr in enumerate(probs))
        ans["choice"] = p.names[best]
    else:
        ans["answer"] = p.names[best]
    return ans


def build_response(model: str, prepared: list, rows: list, cached: list, temperature: float, echo_ids: bool) -> dict:
    answers = {}
    for p, row in zip(prepared, rows):
        a = score_question(p, row, temperature)
        if echo_ids:
            a["prompt_token_ids"] = p.prompt
        answers[p.id] = a
    pt = sum(len(p.prompt) for p in prepared)
    return {"object": "decision", "model": model, "prompt_format_version": PROMPT_FORMAT_VERSION, "answers": answers,
            "usage": {"prompt_tokens": pt, "completion_tokens": 0, "total_tokens": pt, "prompt_tokens_details": {"cached_tokens": int(sum(cached))}}}
