"""Chat templates and the text pipeline of a reply: stop strings, reasoning split, tool-call extraction.

Templates are HF-compatible Jinja (``chat_template.jinja`` or ``tokenizer_config.json: chat_template``), rendered in a
sandbox with ``tojson`` / ``raise_exception`` / ``strftime_now`` as HF provides them (reference crates/server/src/
template.rs:1-9, chat_format.rs:1-16).  The reply pipeline is StreamDecoder -> ReasoningSplitter -> ToolSplitter ->
StopMatcher (reference crates/server/src/http.rs:950-..., reasoning.rs:1-7, tools.rs).
"""
from __future__ import annotations

import json
import os
import time

from jinja2 import TemplateError
from jinja2.sandbox import ImmutableSandboxedEnvironment

CHATML = (
    "{%- for m in messages %}{{ '<|im_start|>' + m['role'] + '\\n' + m['content'] + '<|im_end|>\\n' }}{%- endfor %}"
    "{%- if add_generation_prompt %}{{ '<|im_start|>assistant\\n' }}{%- if enable_thinking is defined and enable_thinking is false %}"
    "{{ '<think>\\n\\n</think>\\n\\n' }}{%- endif %}{%- endif %}"
)


class TemplateRefused(ValueError):
    pass


def _raise(msg):
    raise TemplateRefused(str(msg))


class ChatFormat:
    def __init__(self, template: str = CHATML, bos_token: str = "", eos_token: str = "", think_open: str = "<think>", think_close: str = "</think>",
                 tool_open: str = "<tool_call>", tool_close: str = "</tool_call>"):
        env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)
        env.filters["tojson"] = lambda v, indent=None, ensure_ascii=False, **kw: json.dumps(v, indent=indent, ensure_ascii=ensure_ascii)
        env.globals["raise_exception"] = _raise
        env.globals["strftime_now"] = lambda fmt: time.strftime(fmt)
        try:
            self.template = env.from_string(template)
        except TemplateError as e:
            raise TemplateRefused(f"chat template does not compile: {e}")
        self.bos_token, self.eos_token = bos_token, eos_token
        self.think_open, self.think_close, self.tool_open, self.tool_close = think_open, think_close, tool_open, tool_close

    @staticmethod
    def from_dir(folder: str | None) -> "ChatFormat":
        if folder:
            p = os.path.join(folder, "chat_template.jinja")
            cfgp = os.path.join(folder, "tokenizer_config.json")
            cfg = json.load(open(cfgp, encoding="utf-8")) if os.path.exists(cfgp) else {}
            tok = lambda k: (cfg.get(k) if isinstance(cfg.get(k), str) else (cfg.get(k) or {}).get("content", "")) or ""  # noqa: E731
            if os.path.exists(p):
                return ChatFormat(open(p, encoding="utf-8").read(), tok("bos_token"), tok("eos_token"))
            if isinstance(cfg.get("chat_template"), str):
                return ChatFormat(cfg["chat_template"], tok("bos_token"), tok("eos_token"))
        return ChatFormat()

    def render(self, messages: list, tools=None, add_generation_prompt: bool = True, **kwargs) -> str:
        try:
            return self.template.render(messages=messages, tools=tools, add_generation_prompt=add_generation_prompt, bos_token=self.bos_token,
                                        eos_token=self.eos_token, **kwargs)
        except TemplateRefused:
            raise
        except Exception as e:  # a template error is the request's problem, never the server's
            raise TemplateRefused(f"chat template failed: {e.__class__.__name__}: {e}")


class StopMatcher:
    """Holds back the longest tail that could still become a stop string; `push` returns (text safe to emit, stopped)."""

    def __init__(self, stops):
        self.stops = [s for s in stops if s]
        self.hold = ""
        self.keep = max((len(s) for s in self.stops), default=0) - 1

    def push(self, text: str):
        if not self.stops:
            return text, False
        buf = self.hold + text
        cut = min((i for i in (buf.find(s) for s in self.stops) if i >= 0), default=-1)
        if cut >= 0:
            self.hold = ""
            return buf[:cut], True
        n = 0
        for k in range(min(self.keep, len(buf)), 0, -1):   # longest suffix that is a proper prefix of some stop string
            if any(s.startswith(buf[-k:]) for s in self.stops):
                n = k
                break
        self.hold = buf[len(buf) - n:] if n else ""
        return buf[:len(buf) - n] if n else buf, False

    def flush(self) -> str:
        t, self.hold = self.hold, ""
        return t


class ReasoningSplitter:
    """Routes text between <think> ... </think> to the reasoning channel.  `started_inside` is for templates that open the block in
    the generation prompt.  push() -> (content, reasoning)."""

    def __init__(self, open_tag="<think>", close_tag="</think>", started_inside=False):
        self.open, self.close = open_tag, close_tag
        self.inside = started_inside
        self.done = False
        self.buf = ""
        self.reasoning_chars = 0

    def push(self, text: str):
        content, reasoning = "", ""
        self.buf += text
        while self.buf:
            if self.done:
                content += self.buf
                self.buf = ""
                break
            tag = self.close if self.inside else self.open
            i = self.buf.find(tag)
            if i >= 0:
                head, self.buf = self.buf[:i], self.buf[i + len(tag):]
                if self.inside:
                    reasoning += head
                    self.inside, self.done = False, True
                    self.buf = self.buf.lstrip("\n") if self.buf else self.buf
                else:
                    content += head
                    self.inside = True
                continue
            if not self.inside and content == "" and self.buf.strip() and not self.open.startswith(self.buf.lstrip()[:len(self.open)]):
                self.done = True      # the reply did not start with a reasoning block: there will be none
                continue
            hold = 0
            for k in range(min(len(tag) - 1, len(self.buf)), 0, -1):
                if tag.startswith(self.buf[-k:]):
                    hold = k
                    break
            emit, self.buf = self.buf[:len(self.buf) - hold], self.buf[len(self.buf) - hold:]
            if self.inside:
                reasoning += emit
            else:
                content += emit
            break
        self.reasoning_chars += len(reasoning)
        return content, reasoning

    def flush(self):
        t, self.buf = self.buf, ""
        return ("", t) if self.inside else (t, "")


def extract_tool_calls(text: str, open_tag="<tool_call>", close_tag="</tool_call>"):
    """(text without the call blocks, [OpenAI tool_calls]) for Hermes-style ``<tool_call>{"name":..., "arguments":...}</tool_call>``."""
    calls, out, pos = [], "", 0
    while True:
        i = text.find(open_tag, pos)
        if i < 0:
            out += text[pos:]
            break
        j = text.find(close_tag, i)
        if j < 0:
            out += text[pos:]
            break
        out += text[pos:i]
        blob = text[i + len(open_tag):j].strip()
        try:
            obj = json.loads(blob)
            args = obj.get("arguments", {})
            calls.append({"id": f"call_{len(calls)}_{abs(hash(blob)) % 10 ** 8}", "type": "function",
                          "function": {"name": str(obj.get("name", "")), "arguments": args if isinstance(args, str) else json.dumps(args)}})
        except (json.JSONDecodeError, AttributeError):
            out += text[i:j + len(close_tag)]     # not a well-formed call: leave it in the text
        pos = j + len(close_tag)
    return out.strip() if calls else out, calls
