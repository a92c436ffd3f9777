"""Chat formats by model family: everything the HTTP layer needs to know about how one family talks, behind one interface, found through a
registry (reference crates/server/src/chat_format.rs:1-22, formats/mod.rs:14-16).  A format binds the Jinja template's conventions to the
request path: whether a rendered prompt ends inside an open reasoning block and what closes it, which generated tokens open a new turn (and
so end the reply), how the model writes a tool call (markers, block syntax, and how argument values are typed from the request's schemas),
which reasoning controls a request may use (`reasoning_capabilities`), and whether the family takes images.

Lookup key: the model folder's `config.json` — `architectures[0]`, else `model_type` — matched exactly against the entries' names;
`--chat-format ID` names an entry directly.  A model nothing matches is refused with the list of what is registered, never given another
family's format.  The packs this repository's quantizer writes (`model_type` rexl3_*) carry no family template, so they map to the
"chatml" entry (the built-in ChatML template with the function-block-free JSON tool syntax).

Adding a family: subclass `FamilyFormat`, set `id` / `names`, override what differs, append the class to `BUILTIN`.
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass, field

from .text import CHATML, ChatFormat, TemplateRefused


# ====================================================================================================== tool schemas and value typing
class ToolSchemas:
    """Parameter schemas by function name, from the request's `tools` (reference crates/server/src/tools.rs:35-70)."""

    def __init__(self, params: dict):
        self.params = params          # function name -> its `parameters` schema (or {})

    @staticmethod
    def from_request(tools, tool_choice=None) -> "ToolSchemas | None":
        if not tools or tool_choice == "none":
            return None
        params = {}
        for t in tools:
            f = t.get("function", t) if isinstance(t, dict) else None
            if isinstance(f, dict) and isinstance(f.get("name"), str):
                params[f["name"]] = f.get("parameters") if isinstance(f.get("parameters"), dict) else {}
        return ToolSchemas(params)

    def resolve_name(self, func: str) -> "str | None":
        """The declared spelling of `func`: exact, else case-insensitive, else its last `::` segment."""
        if func in self.params:
            return func
        low = func.lower()
        bare = low.rsplit("::", 1)[-1]
        for k in self.params:
            if k.lower() in (low, bare):
                return k
        return None

    def param_schema(self, func: str, key: str):
        root = self.params.get(func) or {}
        props = root.get("properties")
        return (props.get(key) if isinstance(props, dict) else None), root


def _deref(schema, root, depth=0):
    while isinstance(schema, dict) and isinstance(schema.get("$ref"), str) and depth < 8:
        node = root
        ref = schema["$ref"]
        if not ref.startswith("#/"):
            return schema
        for part in ref[2:].split("/"):
            node = node.get(part) if isinstance(node, dict) else None
        schema, depth = node, depth + 1
    return schema


def _types_of(schema, root) -> list:
    """The JSON types a schema admits, in the order they should be tried (unions and enums read; `$ref` followed)."""
    schema = _deref(schema, root)
    if not isinstance(schema, dict):
        return []
    t = schema.get("type")
    out = list(t) if isinstance(t, list) else ([t] if isinstance(t, str) else [])
    for key in ("anyOf", "oneOf"):
        for alt in schema.get(key) or []:
            out += _types_of(alt, root)
    if not out and isinstance(schema.get("enum"), list):
        for v in schema["enum"]:
            out.append({bool: "boolean", int: "integer", float: "number", str: "string", type(None): "null"}.get(type(v), "object"))
    return out


def typed_value(text: str, schema, root):
    """A tool-call argument written as text -> the JSON value its declared schema means.  A string stays verbatim where the schema admits a
    string and nothing narrower matches; numbers, booleans, null, arrays and objects are read as JSON when the schema asks for them; an
    undeclared parameter is read as JSON when it parses and kept as a string otherwise."""
    types = _types_of(schema, root)
    raw = text.strip()
    if not types:
        try:
            return json.loads(raw)
        except ValueError:
            return text
    for t in types:
        if t == "string":
            continue
        try:
            v = json.loads(raw)
        except ValueError:
            if t == "boolean" and raw.lower() in ("true", "false"):
                return raw.lower() == "true"
            continue
        if ((t == "integer" and isinstance(v, int) and not isinstance(v, bool)) or (t == "number" and isinstance(v, (int, float)) and not isinstance(v, bool))
                or (t == "boolean" and isinstance(v, bool)) or (t == "null" and v is None) or (t == "array" and isinstance(v, list))
                or (t == "object" and isinstance(v, dict))):
            return v
    return text if "string" in types else raw


# ====================================================================================================== tool syntaxes
@dataclass(frozen=True)
class ToolSyntax:
    """How a family writes tool calls in its reply: the text that opens and closes one call (or one group of calls) and the reader of what
    is between them.  `parse(block, schemas)` returns a list of (name, arguments dict), or None when the block is not a call the family's
    template would produce (the block then stays in the visible text instead of running a tool with half its arguments)."""
    id: str
    open: str
    close: str
    parse: object


def _parse_json_block(block: str, schemas):
    try:
        obj = json.loads(block.strip())
    except ValueError:
        return None
    if not isinstance(obj, dict) or not isinstance(obj.get("name"), str) or not obj["name"]:
        return None
    args = obj.get("arguments", {})
    if isinstance(args, str):
        try:
            args = json.loads(args)
        except ValueError:
            return None
    return [(obj["name"], args)] if isinstance(args, dict) else None


_FUNC_RE = re.compile(r"\s*<function=([^>\s]+)>(.*?)</function>\s*", re.S)
_PARAM_RE = re.compile(r"\s*<parameter=([^>\s]+)>\n?(.*?)\n?</parameter>", re.S)


def _parse_function_block(block: str, schemas):
    """`<function=NAME><parameter=KEY>\\nVALUE\\n</parameter></function>`; values are text, typed from the request's schema."""
    m = _FUNC_RE.fullmatch(block)
    if not m:
        return None
    name, body = m.group(1), m.group(2)
    declared = schemas.resolve_name(name) if schemas else None
    args, pos = {}, 0
    body = body.strip("\n")
    while pos < len(body):
        pm = _PARAM_RE.match(body, pos)
        if not pm:
            if body[pos:].strip():
                return None
            break
        schema, root = schemas.param_schema(declared, pm.group(1)) if (schemas and declared) else (None, {})
        args[pm.group(1)] = typed_value(pm.group(2), schema, root)
        pos = pm.end()
    return [(declared or name, args)]


def _parse_arg_pairs(block: str, schemas):
    """`NAME<arg_key>K</arg_key><arg_value>V</arg_value>...` (whitespace between the tags tolerated; a string value is taken exactly as
    written between the value tags).  Reference crates/server/src/formats/glm/tools.rs:1-20."""
    ko, kc, vo, vc = "<arg_key>", "</arg_key>", "<arg_value>", "</arg_value>"
    end = block.find(ko)
    name = (block if end < 0 else block[:end]).strip()
    if not name or any(c.isspace() for c in name) or "<" in name or ">" in name:
        return None
    declared = schemas.resolve_name(name) if schemas else None
    rest, args = ("" if end < 0 else block[end:]), {}
    while True:
        rest = rest.lstrip()
        if not rest:
            break
        if not rest.startswith(ko):
            return None
        i = rest.find(kc)
        if i < 0:
            return None
        key = rest[len(ko):i].strip()
        if not key or "<" in key or ">" in key:
            return None
        rest = rest[i + len(kc):].lstrip()
        if not rest.startswith(vo):
            return None
        j = rest.find(vc)
        if j < 0:
            return None
        schema, root = schemas.param_schema(declared, key) if (schemas and declared) else (None, {})
        args[key] = typed_value(rest[len(vo):j], schema, root)
        rest = rest[j + len(vc):]
    return [(declared or name, args)]


_DSML = "｜DSML｜"
_INVOKE_RE = re.compile(r"\s*<" + _DSML + r" invoke name=\"([^\"]+)\">(.*?)</" + _DSML + r" invoke>\s*", re.S)
_DPARAM_RE = re.compile(r"\s*<" + _DSML + r" parameter name=\"([^\"]+)\" string=\"(true|false)\">(.*?)</" + _DSML + r" parameter>", re.S)


def _parse_dsml(block: str, schemas):
    """One `<|DSML| calls>` group: `<|DSML| invoke name="F"><|DSML| parameter name="K" string="true|false">V</...></...>` repeated.
    `string="true"` values are verbatim strings; the others are JSON."""
    calls, pos = [], 0
    while pos < len(block):
        m = _INVOKE_RE.match(block, pos)
        if not m:
            if block[pos:].strip():
                return None
            break
        args, p, body = {}, 0, m.group(2)
        while p < len(body):
            pm = _DPARAM_RE.match(body, p)
            if not pm:
                if body[p:].strip():
                    return None
                break
            if pm.group(2) == "true":
                args[pm.group(1)] = pm.group(3)
            else:
                try:
                    args[pm.group(1)] = json.loads(pm.group(3))
                except ValueError:
                    return None
            p = pm.end()
        name = m.group(1)
        calls.append(((schemas.resolve_name(name) if schemas else None) or name, args))
        pos = m.end()
    return calls or None


JSON_TOOL_SYNTAX = ToolSyntax("json", "<tool_call>", "</tool_call>", _parse_json_block)
FUNCTION_BLOCK_TOOL_SYNTAX = ToolSyntax("function_block", "<tool_call>", "</tool_call>", _parse_function_block)
ARG_PAIRS_TOOL_SYNTAX = ToolSyntax("arg_pairs", "<tool_call>", "</tool_call>", _parse_arg_pairs)
DSML_TOOL_SYNTAX = ToolSyntax("dsml", "<" + _DSML + " calls>", "</" + _DSML + " calls>", _parse_dsml)


def split_tool_calls(text: str, syntax: ToolSyntax, schemas=None):
    """(visible text, [OpenAI tool_calls]) — every well-formed block of the family's syntax becomes calls; anything else stays text."""
    calls, out, pos = [], "", 0
    while True:
        i = text.find(syntax.open, pos)
        j = text.find(syntax.close, i + len(syntax.open)) if i >= 0 else -1
        if i < 0 or j < 0:
            out += text[pos:]
            break
        out += text[pos:i]
        parsed = syntax.parse(text[i + len(syntax.open):j], schemas)
        if parsed is None:
            out += text[i:j + len(syntax.close)]
        else:
            for name, args in parsed:
                blob = json.dumps(args, ensure_ascii=False)
                calls.append({"id": f"call_{len(calls)}_{abs(hash((name, blob))) % 10 ** 8}", "type": "function",
                              "function": {"name": name, "arguments": blob}})
        pos = j + len(syntax.close)
    return (out.strip() if calls else out), calls


def normalize_history(messages: list) -> list:
    """Tool-call history made renderable: `arguments` given as a JSON string becomes an object (templates iterate over it)."""
    out = []
    for m in messages:
        if isinstance(m, dict) and isinstance(m.get("tool_calls"), list):
            m = dict(m)
            fixed = []
            for c in m["tool_calls"]:
                f = c.get("function") if isinstance(c, dict) else None
                if isinstance(f, dict) and isinstance(f.get("arguments"), str):
                    try:
                        c = dict(c, function=dict(f, arguments=json.loads(f["arguments"])))
                    except ValueError:
                        pass
                fixed.append(c)
            m["tool_calls"] = fixed
        out.append(m)
    return out


# ====================================================================================================== reasoning capabilities
@dataclass
class EffortLevel:
    name: str
    thinks: bool = True
    sets: dict = field(default_factory=dict)      # template variables the level sets


@dataclass
class ReasoningCapabilities:
    """What reasoning controls a family's template offers, as data (reference crates/server/src/reasoning_caps.rs:1-20): the request path
    reads only this, never a family name."""
    reasons: bool = True
    open: str = "<think>"
    close: str = "</think>"
    switch: "str | None" = "enable_thinking"      # the boolean template variable that turns thinking on and off
    switch_closes_block: bool = True               # false closes the block in the prompt (else the model thinks anyway: a note is returned)
    levels: list = field(default_factory=list)     # EffortLevel
    effort_var: "str | None" = None                # a template variable that takes the level's name directly
    thinks_by_default: bool = True
    budget: bool = True                            # the engine may force the closing marker after N reasoning tokens
    extra_vars: dict = field(default_factory=dict)  # other kwargs a request may set: name -> "boolean" | "string" | [choices]

    def level(self, name: str):
        return next((lv for lv in self.levels if lv.name == name), None)

    def level_names(self) -> list:
        return [lv.name for lv in self.levels]

    def describe(self) -> dict:
        return dict(reasons=self.reasons, markers=dict(open=self.open, close=self.close), thinking_switch=self.switch,
                    switch_closes_block=self.switch_closes_block, effort_levels=self.level_names(), effort_variable=self.effort_var,
                    template_thinks_by_default=self.thinks_by_default, reasoning_budget=self.budget, variables=sorted(self.extra_vars))


class ControlRefused(ValueError):
    def __init__(self, message: str, param: str):
        super().__init__(message)
        self.param = param


def apply_reasoning_controls(caps: ReasoningCapabilities, kwargs: dict, *, effort=None, thinking=None, default_thinking: str = "off",
                             default_effort=None) -> tuple:
    """The template kwargs a chat request runs with, and a note for the client (or None).

    kwargs: the request's `chat_template_kwargs` (checked here: only variables the family declares).  effort: the top-level
    `reasoning_effort`; thinking: the top-level `thinking` boolean alias of the switch.  default_thinking ("off" | "template") says what
    happens when the request names neither: "off" inserts the switch set to false where the family has a switch that closes the block and
    its template would think by default; "template" inserts nothing.  default_effort: a level a silent request gets (`--default-reasoning-effort`).
    Reference crates/server/src/reasoning_controls.rs:1-60."""
    out, note = {}, None
    allowed = set(caps.extra_vars)
    if caps.switch:
        allowed.add(caps.switch)
    if caps.effort_var:
        allowed.add(caps.effort_var)
    for lv in caps.levels:
        allowed.update(lv.sets)
    for k, v in (kwargs or {}).items():
        if k not in allowed:
            raise ControlRefused(f"chat_template_kwargs.{k} is not a variable this model's template offers "
                                 f"(offered: {', '.join(sorted(allowed)) or 'none'})", "chat_template_kwargs")
        kind = "boolean" if k == caps.switch else caps.extra_vars.get(k)
        if kind == "boolean" and not isinstance(v, bool):
            raise ControlRefused(f"chat_template_kwargs.{k} must be a boolean", "chat_template_kwargs")
        if kind == "string" and not isinstance(v, str):
            raise ControlRefused(f"chat_template_kwargs.{k} must be a string", "chat_template_kwargs")
        if isinstance(kind, (list, tuple)) and v not in kind:
            raise ControlRefused(f"chat_template_kwargs.{k} must be one of {', '.join(map(str, kind))}", "chat_template_kwargs")
        out[k] = v
    if thinking is not None:
        if not isinstance(thinking, bool):
            raise ControlRefused("'thinking' must be a boolean", "thinking")
        if not caps.switch:
            if thinking and not caps.reasons:
                raise ControlRefused("this model does not reason", "thinking")
        elif caps.switch in out and out[caps.switch] != thinking:
            raise ControlRefused(f"'thinking' contradicts chat_template_kwargs.{caps.switch}", "thinking")
        else:
            out[caps.switch] = thinking
    chose = caps.switch in out if caps.switch else False
    if effort is None and not chose and default_effort is not None:
        effort = default_effort
    if effort is not None:
        if not caps.reasons:
            raise ControlRefused("this model does not reason, so it takes no reasoning effort", "reasoning_effort")
        lv = caps.level(effort) if isinstance(effort, str) else None
        if lv is not None:
            for k, v in lv.sets.items():
                if k in out and out[k] != v:
                    raise ControlRefused(f"reasoning_effort '{effort}' sets {k} = {json.dumps(v)}, the request gives {json.dumps(out[k])}",
                                         "reasoning_effort")
                out[k] = v
            if caps.switch and caps.switch not in out:
                out[caps.switch] = lv.thinks
            elif caps.switch and out[caps.switch] != lv.thinks:
                raise ControlRefused(f"reasoning_effort '{effort}' contradicts {caps.switch}", "reasoning_effort")
        elif caps.effort_var and isinstance(effort, str) and (not isinstance(caps.extra_vars.get(caps.effort_var), (list, tuple))
                                                               or effort in caps.extra_vars[caps.effort_var]):
            out[caps.effort_var] = effort
        else:
            names = caps.level_names() or list(caps.extra_vars.get(caps.effort_var) or [])
            raise ControlRefused(f"'reasoning_effort' must be one of {', '.join(names) or '(none: this model has no effort levels)'}", "reasoning_effort")
        chose = True
    if not chose and default_thinking == "off" and caps.switch and caps.switch_closes_block and caps.thinks_by_default:
        out[caps.switch] = False          # the template would open a reasoning block on its own: the server's default turns it off
    if caps.switch and out.get(caps.switch) is False and not caps.switch_closes_block:
        note = "thinking cannot be turned off for this model: its template always opens a reasoning block"
    return out, note


# ====================================================================================================== families
class FamilyFormat(ChatFormat):
    """A family's conventions bound to a template.  Defaults: ChatML framing, `<think>` blocks, JSON tool calls, text only."""
    id = "chatml"
    names: tuple = ("rexl3_dense", "rexl3_hybrid", "rexl3_moe", "rexl3_mla_moe", "Rexl3DenseForCausalLM", "Rexl3HybridForCausalLM", "Rexl3MoEForCausalLM",
                    "Rexl3MlaMoEForCausalLM", "LlamaForCausalLM", "llama", "Qwen3ForCausalLM", "qwen3", "Qwen3MoeForCausalLM",
                    "qwen3_moe")
    tool = JSON_TOOL_SYNTAX
    role_stop_tokens: tuple = ()          # texts that, generated as ONE token, open a new turn and so end the reply
    serves_images = False
    image_part_types: tuple = ()

    def __init__(self, template: "str | None" = None, bos_token: str = "", eos_token: str = ""):
        caps = self.reasoning_capabilities()
        super().__init__(template if template is not None else self.default_template(), bos_token, eos_token, caps.open, caps.close,
                         self.tool.open, self.tool.close)
        self.caps = caps

    @classmethod
    def default_template(cls) -> str:
        return CHATML

    @classmethod
    def reasoning_capabilities(cls) -> ReasoningCapabilities:
        return ReasoningCapabilities(thinks_by_default=False)

    def starts_in_reasoning(self, prompt: str) -> bool:
        """Whether a reply to this rendered prompt begins inside a reasoning block."""
        p = prompt.rstrip("\n")
        return bool(self.caps.open) and p.endswith(self.caps.open)

    def reply_role_stops(self, tok) -> list:
        out = []
        for text in self.role_stop_tokens:
            ids = tok.encode(text)
            if len(ids) == 1:
                out.append(ids[0])
        return out

    def split_tools(self, text: str, tools, tool_choice=None):
        schemas = ToolSchemas.from_request(tools, tool_choice)
        return split_tool_calls(text, self.tool, schemas) if schemas is not None else (text, [])

    def check_media(self, messages: list) -> "str | None":
        """None when every content part can be honoured, else a sentence naming the first one that cannot."""
        for i, m in enumerate(messages):
            c = m.get("content") if isinstance(m, dict) else None
            if isinstance(c, list):
                for part in c:
                    t = part.get("type") if isinstance(part, dict) else None
                    if t in (None, "text"):
                        continue
                    if t in self.image_part_types and self.serves_images:
                        continue
                    return f"messages[{i}] has a '{t}' part; the '{self.id}' chat format on this server takes text only"
        return None

    def render(self, messages: list, tools=None, add_generation_prompt: bool = True, **kwargs) -> str:
        return super().render(normalize_history(messages), tools=tools, add_generation_prompt=add_generation_prompt, **kwargs)


class QwenFormat(FamilyFormat):
    """Qwen3.5-class: `<think>\\n` generation prompt, `<tool_call><function=NAME><parameter=KEY>` calls, `<|vision_start|><|image_pad|>
    <|vision_end|>` images (reference crates/server/src/formats/qwen.rs:1-2)."""
    id = "qwen"
    names = ("Qwen3_5ForConditionalGeneration", "Qwen3_5ForCausalLM", "Qwen3_5MoeForConditionalGeneration", "Qwen3_5MoeForCausalLM", "qwen3_5",
             "qwen3_5_text", "qwen3_5_moe", "qwen3_5_moe_text")
    tool = FUNCTION_BLOCK_TOOL_SYNTAX
    role_stop_tokens = ("<|im_start|>",)
    image_part_types = ("image_url", "image")

    @classmethod
    def default_template(cls) -> str:
        return CHATML.replace("{{ '<|im_start|>assistant\\n' }}{%- if enable_thinking is defined and enable_thinking is false %}"
                              "{{ '<think>\\n\\n</think>\\n\\n' }}{%- endif %}",
                              "{{ '<|im_start|>assistant\\n' }}{%- if enable_thinking is defined and enable_thinking is false %}"
                              "{{ '<think>\\n\\n</think>\\n\\n' }}{%- else %}{{ '<think>\\n' }}{%- endif %}")

    @classmethod
    def reasoning_capabilities(cls) -> ReasoningCapabilities:
        return ReasoningCapabilities(thinks_by_default=True)

    def starts_in_reasoning(self, prompt: str) -> bool:
        return prompt.rstrip("\n").endswith("<think>") and not prompt.endswith("</think>\n\n")


class MimoFormat(QwenFormat):
    """MiMo-V2: the Qwen framing and tool syntax; its vision / audio placeholders are refused (no tower)."""
    id = "mimo"
    names = ("MiMoV2ForCausalLM", "mimo_v2")
    image_part_types = ()


class GlmFormat(FamilyFormat):
    """GLM-5-class: `<tool_call>NAME<arg_key>K</arg_key><arg_value>V</arg_value></tool_call>` calls, `<think>` blocks, thinking on by default."""
    id = "glm5_next"
    names = ("Glm5NextForConditionalGeneration", "glm5_next")
    tool = ARG_PAIRS_TOOL_SYNTAX
    role_stop_tokens = ("<|user|>", "<|observation|>")
    image_part_types = ("image_url", "image")

    @classmethod
    def reasoning_capabilities(cls) -> ReasoningCapabilities:
        return ReasoningCapabilities(thinks_by_default=True)


class BailingFormat(FamilyFormat):
    """Bailing-3.x: `<role>HUMAN|ASSISTANT|...</role>` turns ended by `<|role_end|>`, GLM-shaped tool calls, effort levels through a
    template variable (reference crates/server/src/formats/bailing_moe_v3.rs:1-3)."""
    id = "bailing_moe_v3"
    names = ("BailingMoeV3ForCausalLM", "bailing_hybrid", "bailing_moe_v3")
    tool = ARG_PAIRS_TOOL_SYNTAX
    role_stop_tokens = ("<|role_end|>",)

    @classmethod
    def default_template(cls) -> str:
        return ("{%- for m in messages %}{{ '<role>' + ({'system': 'SYSTEM', 'user': 'HUMAN', 'assistant': 'ASSISTANT', 'tool': 'OBSERVATION'}[m['role']]) "
                "+ '</role>' + m['content'] + '<|role_end|>' }}{%- endfor %}{%- if add_generation_prompt %}{{ '<role>ASSISTANT</role>' }}"
                "{%- if enable_thinking is defined and enable_thinking %}{{ '<think>' }}{%- endif %}{%- endif %}")

    @classmethod
    def reasoning_capabilities(cls) -> ReasoningCapabilities:
        return ReasoningCapabilities(thinks_by_default=False, levels=[EffortLevel("none", False), EffortLevel("low", True, {"thinking_budget": "low"}),
                                                                      EffortLevel("high", True, {"thinking_budget": "high"})],
                                     extra_vars={"thinking_budget": ["low", "high"]})

    def starts_in_reasoning(self, prompt: str) -> bool:
        return prompt.endswith("<think>") or prompt.endswith("<think>\n")


class DeepseekV41Format(FamilyFormat):
    """DeepSeek-V4.1: `<|begin_of_sentence|>` / `<|User|>` / `<|Assistant|>` framing (full-width bars), `<think>` blocks switched by the
    `thinking` variable, DSML tool calls; the template is built in (the family ships none the server trusts).  Reference
    crates/server/src/formats/deepseek_v41.rs:1-2."""
    id = "deepseek_v41"
    names = ("DeepseekV4ForCausalLM", "DeepseekV41ForCausalLM", "DeepseekV41ForConditionalGeneration", "deepseek_v4", "deepseek_v41", "deepseek_v41_text",
             "DeepseekV3ForCausalLM", "deepseek_v3")
    tool = DSML_TOOL_SYNTAX
    role_stop_tokens = ("<｜User｜>",)

    @classmethod
    def default_template(cls) -> str:
        b = "｜"
        return ("{{ '<" + b + "begin▁of▁sentence" + b + ">' }}{%- for m in messages %}{%- if m['role'] == 'system' %}{{ m['content'] }}"
                "{%- elif m['role'] == 'user' %}{{ '<" + b + "User" + b + ">' + m['content'] }}"
                "{%- elif m['role'] == 'assistant' %}{{ '<" + b + "Assistant" + b + "></think>' + m['content'] + '<" + b + "end▁of▁sentence" + b + ">' }}"
                "{%- else %}{{ '<" + b + "User" + b + ">' + m['content'] }}{%- endif %}{%- endfor %}"
                "{%- if add_generation_prompt %}{{ '<" + b + "Assistant" + b + ">' }}{%- if thinking is defined and thinking %}{{ '<think>' }}"
                "{%- else %}{{ '</think>' }}{%- endif %}{%- endif %}")

    @classmethod
    def reasoning_capabilities(cls) -> ReasoningCapabilities:
        return ReasoningCapabilities(switch="thinking", thinks_by_default=False,
                                     levels=[EffortLevel("none", False), EffortLevel("low", True, {"reasoning_effort": "low"}),
                                             EffortLevel("medium", True, {"reasoning_effort": "medium"}), EffortLevel("high", True, {"reasoning_effort": "high"})],
                                     extra_vars={"reasoning_effort": ["low", "medium", "high"]})

    def starts_in_reasoning(self, prompt: str) -> bool:
        return prompt.endswith("<think>")


class NemotronOmniFormat(FamilyFormat):
    """Nemotron-H omni: ChatML-like turns, `<think>` blocks the template ALWAYS opens (the switch is accepted and noted, it cannot close the
    block), JSON tool calls between `<TOOLCALL>` markers, `<image>` placeholders between `<img>`..`</img>`."""
    id = "nemotron_omni"
    names = ("NemotronH_Omni_Reasoning_V3", "nemotron_h_omni", "NemotronHForCausalLM", "nemotron_h")
    tool = ToolSyntax("json_list", "<TOOLCALL>", "</TOOLCALL>",
                      lambda block, schemas: _parse_json_list(block))
    image_part_types = ("image_url", "image")

    @classmethod
    def reasoning_capabilities(cls) -> ReasoningCapabilities:
        return ReasoningCapabilities(switch_closes_block=False, thinks_by_default=True)


def _parse_json_list(block: str):
    try:
        arr = json.loads(block.strip())
    except ValueError:
        return None
    if not isinstance(arr, list) or not arr:
        return None
    out = []
    for obj in arr:
        if not isinstance(obj, dict) or not isinstance(obj.get("name"), str) or not isinstance(obj.get("arguments", {}), dict):
            return None
        out.append((obj["name"], obj.get("arguments", {})))
    return out


class MiniCpmVFormat(QwenFormat):
    """MiniCPM-V 4.x: the Qwen3.5 text framing with `<|image_pad|>` / `<|video_pad|>` placeholders."""
    id = "minicpmv"
    names = ("MiniCPMV4_7ForConditionalGeneration", "minicpmv4_7")
    image_part_types = ("image_url", "image", "video_url", "video")


BUILTIN = (FamilyFormat, QwenFormat, GlmFormat, MimoFormat, NemotronOmniFormat, MiniCpmVFormat, DeepseekV41Format, BailingFormat)


class FormatRefused(ValueError):
    pass


def registered() -> dict:
    return {f.id: list(f.names) for f in BUILTIN}


def find(config: "dict | None", override: "str | None" = None):
    """The family class for a model's `config.json` (or for `--chat-format ID`); raises FormatRefused naming what is registered."""
    if override:
        for f in BUILTIN:
            if f.id == override:
                return f
        raise FormatRefused(f"no chat format is registered as '{override}' (registered: {', '.join(f.id for f in BUILTIN)})")
    config = config or {}
    arch = config.get("architectures")
    key = arch[0] if isinstance(arch, list) and arch and isinstance(arch[0], str) else config.get("model_type")
    if key is None:
        return FamilyFormat
    for f in BUILTIN:
        if key in f.names:
            return f
    listing = "; ".join(f"{f.id}: {', '.join(f.names)}" for f in BUILTIN)
    raise FormatRefused(f"no chat format is registered for '{key}' (pass --chat-format ID to choose one; registered: {listing})")


def open_format(folder: "str | None", override: "str | None" = None) -> FamilyFormat:
    """The chat format of a model folder: the family from config.json (or the override), bound to the folder's own template when it ships
    one (`chat_template.jinja`, else `tokenizer_config.json: chat_template`), else to the family's built-in template."""
    import os
    config, template, bos, eos = None, None, "", ""
    if folder:
        cp = os.path.join(folder, "config.json")
        if os.path.exists(cp):
            with open(cp, encoding="utf-8") as f:
                config = json.load(f)
        tp, tc = os.path.join(folder, "chat_template.jinja"), os.path.join(folder, "tokenizer_config.json")
        cfg = {}
        if os.path.exists(tc):
            with open(tc, encoding="utf-8") as f:
                cfg = json.load(f)
        tok = lambda k: (cfg.get(k) if isinstance(cfg.get(k), str) else (cfg.get(k) or {}).get("content", "")) or ""  # noqa: E731
        bos, eos = tok("bos_token"), tok("eos_token")
        if os.path.exists(tp):
            with open(tp, encoding="utf-8") as f:
                template = f.read()
        elif isinstance(cfg.get("chat_template"), str):
            template = cfg["chat_template"]
    cls = find(config, override)
    try:
        return cls(template, bos, eos)
    except TemplateRefused as e:
        raise FormatRefused(f"the '{cls.id}' chat format cannot use this model's template: {e}")
