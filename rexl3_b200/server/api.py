"""Request parsing and response shaping for the OpenAI-compatible endpoints.

Requests are read field by field.  Unknown fields and unsupported features that would change the output are refused by
name with an OpenAI-shaped 400 instead of being silently ignored; a short list of bookkeeping fields is accepted and
ignored.  Behaviour parity: reference crates/server/src/api.rs:1-4 (policy), :36-44 (stop limits, top_k cap 56),
:86-160 (error shapes, context_length_exceeded), :178-300 (fields), :376-396 (usage object).
"""
from __future__ import annotations

import time
import uuid
from dataclasses import dataclass, field

from ..sampling import Sampling

MAX_STOP_STRINGS = 16
MAX_STOP_BYTES = 1024
TOP_K_CAP = 56
MAX_LOGPROBS = 20

IGNORED_FIELDS = {"user", "metadata", "store", "service_tier", "stream_options", "logit_bias", "presence_penalty", "frequency_penalty",
                  "repetition_penalty", "n", "response_format", "tool_choice", "parallel_tool_calls", "logprobs", "top_logprobs"}
CHAT_FIELDS = {"messages", "model", "temperature", "top_p", "top_k", "min_p", "seed", "max_tokens", "max_completion_tokens", "stop", "stream",
               "stream_options", "skip_special_tokens", "return_token_ids", "draft", "prefix_cache", "prompt_logprobs", "tools",
               "chat_template_kwargs", "max_reasoning_tokens", "reasoning_effort", "thinking"} | IGNORED_FIELDS
COMPLETION_FIELDS = (CHAT_FIELDS - {"messages", "tools", "chat_template_kwargs", "max_reasoning_tokens", "reasoning_effort", "thinking"}) | {"prompt", "echo"}


class ApiError(Exception):
    def __init__(self, status: int, message: str, type_: str = "invalid_request_error", code: str | None = None, param: str | None = None,
                 retry_after: int | None = None):
        super().__init__(message)
        self.status, self.message, self.type, self.code, self.param, self.retry_after = status, message, type_, code, param, retry_after

    def body(self) -> dict:
        return {"error": {"message": self.message, "type": self.type, "code": self.code, "param": self.param}}


def bad(message: str, param: str | None = None, code: str | None = None) -> ApiError:
    return ApiError(400, message, "invalid_request_error", code, param)


@dataclass
class GenDefaults:
    temperature: float = 1.0
    top_p: float = 0.95
    top_k: int = 20

    @staticmethod
    def from_dict(d: dict) -> "GenDefaults":
        g = GenDefaults()
        for k in ("temperature", "top_p", "top_k"):
            if isinstance(d.get(k), (int, float)) and not isinstance(d.get(k), bool):
                setattr(g, k, type(getattr(g, k))(d[k]))
        return g


@dataclass
class Params:
    sampling: Sampling
    max_tokens: int | None = None
    stop: list = field(default_factory=list)
    stream: bool = False
    include_usage: bool = False
    skip_special: bool = True
    seed: int | None = None
    return_token_ids: bool = False
    draft: bool = True
    prefix_cache: bool = True
    prompt_logprobs: int | None = None
    tools: list | None = None
    template_kwargs: dict = field(default_factory=dict)
    max_reasoning_tokens: int | None = None
    reasoning_effort: str | None = None
    thinking: bool | None = None
    tool_choice: object = None
    model: str | None = None


def _num(body, key, lo=None, hi=None, integer=False):
    v = body.get(key)
    if v is None:
        return None
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (integer and not float(v).is_integer()):
        raise bad(f"'{key}' must be {'an integer' if integer else 'a number'}", key)
    if v != v or (lo is not None and v < lo) or (hi is not None and v > hi):
        raise bad(f"'{key}' is out of range", key)
    return int(v) if integer else float(v)


def parse_params(body: dict, allowed: set, defaults: GenDefaults) -> Params:
    if not isinstance(body, dict):
        raise bad("the request body must be a JSON object")
    for k in body:
        if k not in allowed:
            raise bad(f"unknown field '{k}'", k, "unknown_field")
    # features that would change the output and are not implemented: refused by name
    if body.get("n") not in (None, 1):
        raise bad("'n' other than 1 is not supported", "n", "unsupported")
    if body.get("logit_bias"):
        raise bad("'logit_bias' is not supported", "logit_bias", "unsupported")
    for k in ("presence_penalty", "frequency_penalty"):
        if body.get(k) not in (None, 0, 0.0):
            raise bad(f"'{k}' is not supported", k, "unsupported")
    if body.get("repetition_penalty") not in (None, 1, 1.0):
        raise bad("'repetition_penalty' is not supported", "repetition_penalty", "unsupported")
    rf = body.get("response_format")
    if isinstance(rf, dict) and rf.get("type") in ("json_object", "json_schema"):
        raise bad("structured output ('response_format') is not supported", "response_format", "unsupported")
    tc = body.get("tool_choice")
    if tc is not None and tc not in ("auto", "none"):
        raise bad("'tool_choice' must be 'auto' or 'none'", "tool_choice", "unsupported")
    if body.get("parallel_tool_calls"):
        raise bad("'parallel_tool_calls' is not supported", "parallel_tool_calls", "unsupported")
    if body.get("logprobs") not in (None, False, 0) or body.get("top_logprobs") not in (None, 0):
        raise bad("log probabilities of generated tokens are not supported (use 'prompt_logprobs')", "logprobs", "unsupported")

    t = _num(body, "temperature", 0.0, 100.0)
    top_p = _num(body, "top_p", 0.0, 1.0)
    top_k = _num(body, "top_k", -1, 1 << 20, integer=True)
    min_p = _num(body, "min_p", 0.0, 1.0)
    seed = _num(body, "seed", 0, (1 << 63) - 1, integer=True)
    k = defaults.top_k if top_k is None else top_k
    if k <= 0:
        k = TOP_K_CAP
    k = min(k, TOP_K_CAP)
    samp = Sampling(seed=seed or 0, temperature=defaults.temperature if t is None else t, top_k=k,
                    top_p=defaults.top_p if top_p is None else top_p, min_p=0.0 if min_p is None else min_p)
    mt = _num(body, "max_completion_tokens", 1, 1 << 31, integer=True) or _num(body, "max_tokens", 1, 1 << 31, integer=True)
    stop = body.get("stop")
    if stop is None:
        stop = []
    elif isinstance(stop, str):
        stop = [stop]
    if not isinstance(stop, list) or any(not isinstance(s, str) for s in stop):
        raise bad("'stop' must be a string or a list of strings", "stop")
    stop = [s for s in stop if s]
    if len(stop) > MAX_STOP_STRINGS or any(len(s.encode()) > MAX_STOP_BYTES for s in stop):
        raise bad(f"at most {MAX_STOP_STRINGS} stop strings of at most {MAX_STOP_BYTES} bytes", "stop")
    so = body.get("stream_options")
    if so is not None and not isinstance(so, dict):
        raise bad("'stream_options' must be an object", "stream_options")
    pl = body.get("prompt_logprobs")
    if pl is True:
        pl = 1
    if pl is not None and (isinstance(pl, bool) or not isinstance(pl, int) or not 0 <= pl <= MAX_LOGPROBS):
        raise bad(f"'prompt_logprobs' must be an integer in 0..{MAX_LOGPROBS}", "prompt_logprobs")
    tk = body.get("chat_template_kwargs") or {}
    if not isinstance(tk, dict):
        raise bad("'chat_template_kwargs' must be an object", "chat_template_kwargs")
    tools = body.get("tools")
    if tools is not None and (not isinstance(tools, list) or any(not isinstance(x, dict) for x in tools)):
        raise bad("'tools' must be a list of objects", "tools")
    for key in ("stream", "skip_special_tokens", "return_token_ids", "draft", "prefix_cache"):
        if body.get(key) is not None and not isinstance(body[key], bool):
            raise bad(f"'{key}' must be a boolean", key)
    return Params(sampling=samp, max_tokens=mt, stop=stop, stream=bool(body.get("stream", False)),
                  include_usage=bool((so or {}).get("include_usage", False)), skip_special=body.get("skip_special_tokens", True) is not False,
                  seed=seed, return_token_ids=bool(body.get("return_token_ids", False)), draft=body.get("draft", True) is not False,
                  prefix_cache=body.get("prefix_cache", True) is not False, prompt_logprobs=pl, tools=tools, template_kwargs=tk,
                  max_reasoning_tokens=_num(body, "max_reasoning_tokens", 0, 1 << 31, integer=True),
                  reasoning_effort=_effort(body), thinking=_thinking(body), tool_choice=body.get("tool_choice"),
                  model=body.get("model") if isinstance(body.get("model"), str) else None)


def _effort(body: dict):
    v = body.get("reasoning_effort")
    if v is not None and not isinstance(v, str):
        raise bad("'reasoning_effort' must be a string", "reasoning_effort")
    return v


def _thinking(body: dict):
    v = body.get("thinking")
    if v is not None and not isinstance(v, bool):
        raise bad("'thinking' must be a boolean", "thinking")
    return v


def parse_messages(body: dict, image_hook=None) -> list:
    """`image_hook(part) -> str`: called for every image part when the server has a vision tower; what it returns (the chat format's image
    placeholder) takes the part's place in the message text.  Without a hook an image part is refused by name."""
    msgs = body.get("messages")
    if not isinstance(msgs, list) or not msgs:
        raise bad("'messages' must be a non-empty list", "messages")
    out = []
    for i, m in enumerate(msgs):
        if not isinstance(m, dict) or not isinstance(m.get("role"), str):
            raise bad(f"messages[{i}] must be an object with a 'role'", "messages")
        c = m.get("content")
        if isinstance(c, list):
            parts = []
            for part in c:
                if not isinstance(part, dict):
                    raise bad(f"messages[{i}].content parts must be objects", "messages")
                ty = part.get("type")
                if ty == "text":
                    parts.append(str(part.get("text", "")))
                elif ty in ("image_url", "image"):
                    if image_hook is None:
                        raise bad("image input is not supported by this model", "messages", "unsupported")
                    parts.append(image_hook(part))
                else:
                    raise bad(f"content part type '{ty}' is not supported", "messages", "unsupported")
            c = "".join(parts)
        elif c is None:
            c = ""
        elif not isinstance(c, str):
            raise bad(f"messages[{i}].content must be a string or a list of parts", "messages")
        mm = dict(m)
        mm["content"] = c
        out.append(mm)
    return out


def usage_object(u: dict, reasoning_tokens: int = 0) -> dict:
    return {"prompt_tokens": u.get("prompt_tokens", 0), "completion_tokens": u.get("completion_tokens", 0),
            "total_tokens": u.get("total_tokens", 0), "prompt_tokens_details": {"cached_tokens": u.get("cached_tokens", 0)},
            "completion_tokens_details": {"reasoning_tokens": reasoning_tokens}, "spec": u.get("spec", {"drafted": 0, "accepted": 0, "rounds": 0})}


def new_id(prefix: str) -> str:
    return f"{prefix}-{uuid.uuid4().hex[:24]}"


def finish_reason(reason: str) -> str:
    return {"stop": "stop", "length": "length", "cancelled": "stop", "deadline": "length"}.get(reason, "stop")


def chat_completion(rid, model, text, reasoning, tool_calls, reason, usage, fingerprint, token_ids=None, prompt_logprobs=None) -> dict:
    msg = {"role": "assistant", "content": text}
    if reasoning:
        msg["reasoning_content"] = reasoning
    if tool_calls:
        msg["tool_calls"] = tool_calls
    choice = {"index": 0, "message": msg, "finish_reason": "tool_calls" if tool_calls else finish_reason(reason)}
    if token_ids is not None:
        choice["token_ids"] = token_ids
    out = {"id": rid, "object": "chat.completion", "created": int(time.time()), "model": model, "choices": [choice], "usage": usage,
           "system_fingerprint": fingerprint, "prompt_tokens_count": usage["prompt_tokens"]}
    if prompt_logprobs is not None:
        out["prompt_logprobs"] = prompt_logprobs
    return out


def chat_chunk(rid, model, delta: dict, reason=None, fingerprint=None, usage=None) -> dict:
    out = {"id": rid, "object": "chat.completion.chunk", "created": int(time.time()), "model": model, "system_fingerprint": fingerprint,
           "choices": [] if usage is not None and not delta and reason is None else [{"index": 0, "delta": delta, "finish_reason": reason}]}
    if usage is not None:
        out["usage"] = usage
    return out


def text_completion(rid, model, text, reason, usage, fingerprint, stream_chunk=False) -> dict:
    out = {"id": rid, "object": "text_completion", "created": int(time.time()), "model": model, "system_fingerprint": fingerprint,
           "choices": [{"index": 0, "text": text, "finish_reason": None if (stream_chunk and reason is None) else finish_reason(reason or "stop"),
                        "logprobs": None}]}
    if usage is not None:
        out["usage"] = usage
    return out
