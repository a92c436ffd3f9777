"""OpenAI-compatible HTTP surface (ASGI / Starlette).

Routes (reference crates/server/src/http.rs:229-243): GET /health/live, /health, /health/ready, /v1/health, /v1/models,
/metrics; POST /v1/chat/completions (SSE when ``stream``), /v1/completions, /v1/chat/completions/render, /tokenize.
Errors are OpenAI-shaped; 429 / 503 carry Retry-After.  The default seed is sha256 of the prompt tokens: same conversation,
same reply.
"""
from __future__ import annotations

import asyncio
import json

from starlette.applications import Starlette
from starlette.requests import Request as HttpRequest
from starlette.responses import JSONResponse, PlainTextResponse, StreamingResponse
from starlette.routing import Route

from ..engine import Request
from ..sampling import seed_for
from . import api
from .runtime import EngineHandle
from . import budget, formats
from .text import ChatFormat, ReasoningSplitter, StopMatcher, TemplateRefused, extract_tool_calls
from .tokenizer import Tok


class AppState:
    def __init__(self, handle: EngineHandle, tok: Tok, fmt: ChatFormat, model_name: str, max_model_len: int, aliases=(), defaults=None,
                 default_max_tokens: int = 512, fingerprint: str = "rexl3-b200", max_body_bytes: int = 64 << 20, info: dict | None = None,
                 limits=None, default_thinking: str = "template", default_effort: str | None = None, vision=None):
        self.handle, self.tok, self.fmt = handle, tok, fmt
        self.vision = vision              # server.media.VisionIngress: image parts of chat messages are decoded, encoded and laid into the prompt
        self.model_name, self.aliases = model_name, set(aliases)
        self.max_model_len, self.default_max_tokens = max_model_len, default_max_tokens
        self.defaults = defaults or api.GenDefaults()
        self.fingerprint, self.max_body_bytes = fingerprint, max_body_bytes
        self.info = info or {}
        # request budgets (body, JSON nodes / depth, rendered prompt, preparation slots, priced tokenizer memory)
        self.limits = limits or budget.Limits.for_window(max_model_len)
        self.max_body_bytes = min(self.max_body_bytes, self.limits.body_bytes)
        self.prep_gate = budget.PreparationGate(self.limits.preparation_concurrency, self.limits.preparation_queue)
        self.tok_gate = budget.TokenizerGate(self.limits.processing_reserve_bytes, self.limits.tokenizer_wait_s)
        # what a chat request that names neither the thinking switch nor an effort level gets ("off" | "template"), and an optional default level
        self.default_thinking, self.default_effort = default_thinking, default_effort
        self.family = isinstance(fmt, formats.FamilyFormat)
        self.role_stops = tuple(fmt.reply_role_stops(tok)) if self.family else ()


def _err(e: api.ApiError) -> JSONResponse:
    h = {"Retry-After": str(e.retry_after)} if e.retry_after else None
    return JSONResponse(e.body(), status_code=e.status, headers=h)


async def _json_body(request: HttpRequest, st: AppState) -> dict:
    raw = await request.body()
    if len(raw) > st.max_body_bytes:
        raise api.ApiError(413, "request body too large", code="body_too_large")
    try:
        body = json.loads(raw)
    except (json.JSONDecodeError, UnicodeDecodeError, RecursionError):
        raise api.bad("the request body is not valid JSON")
    try:
        budget.check_json(body, st.limits)
    except budget.BudgetRefused as e:
        raise _budget_error(e)
    return body


def _budget_error(e: "budget.BudgetRefused") -> api.ApiError:
    return api.ApiError(e.status, str(e), "invalid_request_error" if e.status == 413 else "rate_limit_error", e.code, retry_after=e.retry_after)


def _encode(st: AppState, text: str) -> list:
    """Tokenize under the request budgets: the rendered-size cap, then the priced tokenizer memory."""
    try:
        n = budget.check_rendered(text, st.limits)
        with st.tok_gate.charge(n):
            return st.tok.encode(text)
    except budget.BudgetRefused as e:
        raise _budget_error(e)


def _check_model(st: AppState, p: api.Params) -> None:
    if p.model and p.model != st.model_name and p.model not in st.aliases:
        raise api.ApiError(404, f"model '{p.model}' is not served here", code="model_not_found", param="model")


def _ready_or_503(st: AppState) -> None:
    s = st.handle.state
    if s not in ("ready", "degraded"):
        raise api.ApiError(503, f"engine is {s}", "service_unavailable", s, retry_after=5)


def _make_request(st: AppState, ids: list, p: api.Params, rid: str, prompt_text: str = "") -> Request:
    if not ids:
        raise api.bad("the prompt is empty")
    limit = st.max_model_len
    if len(ids) >= limit:
        raise api.ApiError(400, f"the prompt has {len(ids)} tokens, the context window holds {limit}", code="context_length_exceeded", param="messages")
    room = limit - len(ids)
    max_new = min(room, p.max_tokens if p.max_tokens is not None else st.default_max_tokens)
    samp = p.sampling
    if p.seed is None and samp.temperature > 0:
        samp = samp.with_seed(seed_for(ids, 0))
    stop_ids = tuple(st.tok.eos_ids) + tuple(t for t in st.role_stops if t not in st.tok.eos_ids)     # a generated role token opens a new turn
    req = Request(rid, ids, max_new, samp, stop_ids, draft=p.draft, prefix_cache=p.prefix_cache, media=getattr(p, "media", None))
    if getattr(p, "max_reasoning_tokens", None) is not None and st.fmt.think_close:
        # reasoning budget: the engine forces the closing tag once that many tokens were spent inside the thinking block
        req.reasoning_budget = int(p.max_reasoning_tokens)
        req.think_close_ids = tuple(st.tok.encode(st.fmt.think_close))
        req.think_open_ids = tuple(st.tok.encode(st.fmt.think_open)) if st.fmt.think_open else ()
        req.reasoning_open = _starts_in_reasoning(st, prompt_text)
    return req


def _starts_in_reasoning(st: AppState, prompt_text: str) -> bool:
    if st.family:
        return st.fmt.starts_in_reasoning(prompt_text)
    return bool(st.fmt.think_open) and prompt_text.rstrip().endswith(st.fmt.think_open)


class _Reply:
    """Token ids -> text deltas through the decoder, the reasoning split and the stop matcher."""

    def __init__(self, st: AppState, p: api.Params, chat: bool, prompt_text: str = ""):
        self.dec = st.tok.stream(p.skip_special)
        self.stop = StopMatcher(p.stop)
        self.reason = ReasoningSplitter(st.fmt.think_open, st.fmt.think_close, started_inside=_starts_in_reasoning(st, prompt_text)) if chat else None
        self.ids, self.text, self.reasoning = [], "", ""
        self.stopped = False
        self.eos = set(st.tok.eos_ids) | set(st.role_stops)

    def push(self, ids):
        """-> (content delta, reasoning delta)"""
        if self.stopped:
            return "", ""
        self.ids.extend(ids)
        piece = self.dec.push([i for i in ids if i not in self.eos])
        return self._route(piece)

    def _route(self, piece):
        content, reasoning = (piece, "") if self.reason is None else self.reason.push(piece)
        if content:
            content, hit = self.stop.push(content)
            self.stopped = hit
        self.text += content
        self.reasoning += reasoning
        return content, reasoning

    def finish(self):
        if self.stopped:
            return "", ""
        c, r = self._route(self.dec.flush())
        if self.reason is not None:
            c2, r2 = self.reason.flush()
            c2, hit = self.stop.push(c2) if c2 else ("", False)
            c, r = c + c2, r + r2
            self.text += c2
            self.reasoning += r2
        tail = "" if self.stopped else self.stop.flush()
        self.text += tail
        return c + tail, r


async def _collect(st: AppState, ticket, reply: _Reply):
    """Drive one request to its end (non-streaming).  Returns (reason, usage)."""
    while True:
        msg = await ticket.out.get()
        if msg[0] == "tokens":
            reply.push(msg[1])
            if reply.stopped:
                st.handle.cancel(ticket.id)
        elif msg[0] == "done":
            reply.finish()
            return ("stop" if reply.stopped else msg[1]), msg[2]
        elif msg[0] == "refused":
            code = msg[1]
            raise api.ApiError(400, msg[2], code="context_length_exceeded" if code == "context_length_exceeded" else None)
        else:
            raise api.ApiError(500, str(msg[1]), "server_error", "engine_error")


def _sse(obj) -> bytes:
    return b"data: " + json.dumps(obj, ensure_ascii=False).encode() + b"\n\n"


def build_app(st: AppState) -> Starlette:
    async def live(request):
        return JSONResponse({"status": "ok"})

    async def health(request):
        s = st.handle.state
        ok = s in ("ready",)
        body = {"status": s}
        if st.handle.error:
            body["error"] = st.handle.error
        return JSONResponse(body, status_code=200 if ok else 503)

    async def models(request):
        m = {"id": st.model_name, "object": "model", "owned_by": "rexl3-b200", "max_model_len": st.max_model_len,
             "configured_max_model_len": st.max_model_len, "aliases": sorted(st.aliases)}
        m.update({k: (v() if callable(v) else v) for k, v in st.info.items()})
        return JSONResponse({"object": "list", "data": [m]})

    async def metrics(request):
        from ..utils import loadstats
        m = st.handle.metrics
        m.set("tokenizer_gate_bytes_in_use", st.tok_gate.in_use())
        m.set("tokenizer_gate_bytes_capacity", st.tok_gate.capacity)
        m.set("tokenizer_gate_waited_total", st.tok_gate.waited)
        m.set("tokenizer_gate_refused_total", st.tok_gate.refused)
        m.set("preparation_refused_total", st.prep_gate.refused)
        return PlainTextResponse(m.render() + loadstats.render(), media_type="text/plain; version=0.0.4")

    async def tokenize(request):
        try:
            body = await _json_body(request, st)
            text = body.get("prompt", body.get("text"))
            if not isinstance(text, str):
                raise api.bad("'prompt' must be a string", "prompt")
            ids = st.tok.encode(text)
            return JSONResponse({"tokens": ids, "count": len(ids), "max_model_len": st.max_model_len})
        except api.ApiError as e:
            return _err(e)

    async def decisions(request):
        from . import decisions as dec
        from ..sched import AdmitError
        try:
            body = await _json_body(request, st)
            if isinstance(body, dict) and body.get("model") not in (None, st.model_name) and body.get("model") not in st.aliases:
                raise api.ApiError(404, f"model {body.get('model')!r} is not served", code="model_not_found", param="model")
            _ready_or_503(st)
            try:
                prepared, temp, echo = dec.prepare(body, st.tok, st.fmt, st.max_model_len)
            except TemplateRefused as e:
                raise api.bad(str(e), "input", "template_error")
            loop = asyncio.get_running_loop()
            rows = []
            for p_ in prepared:
                try:
                    rows.append(await st.handle.score(p_.prompt, loop))
                except AdmitError as e:
                    if e.kind == "NoSlot":
                        raise api.ApiError(503, "every sequence slot is busy; retry", "server_error", "overloaded", retry_after=1)
                    raise api.ApiError(400, str(e), code="context_length_exceeded")
                except RuntimeError as e:
                    raise api.ApiError(503, f"engine unavailable: {e}", "server_error", "engine_unavailable")
            return JSONResponse(dec.build_response(st.model_name, prepared, rows, [0] * len(rows), temp, echo))
        except api.ApiError as e:
            return _err(e)

    def render_chat(body, p):
        """-> (prompt text, token ids, note for the client or None)"""
        images, hook = [], None
        if st.vision is not None:
            from .media import MediaError

            def hook(part):
                if len(images) >= st.vision.max_images:
                    raise api.bad(f"more than {st.vision.max_images} images in one request", "messages", "too_many_images")
                try:
                    images.append(st.vision.decode(part))
                except MediaError as e:
                    raise api.bad(str(e), "messages", e.code)
                return st.vision.placeholder_text
        msgs = api.parse_messages(body, hook)
        kwargs, note = p.template_kwargs, None
        if st.family:
            refusal = st.fmt.check_media(msgs)
            if refusal:
                raise api.bad(refusal, "messages", "unsupported_media")
            try:
                kwargs, note = formats.apply_reasoning_controls(st.fmt.caps, p.template_kwargs, effort=p.reasoning_effort, thinking=p.thinking,
                                                                default_thinking=st.default_thinking, default_effort=st.default_effort)
            except formats.ControlRefused as e:
                raise api.bad(str(e), e.param, "reasoning_control")
        elif p.reasoning_effort is not None or p.thinking is not None:
            raise api.bad("this server's chat format declares no reasoning controls", "reasoning_effort", "reasoning_control")
        try:
            text = st.fmt.render(msgs, tools=p.tools, add_generation_prompt=True, **kwargs)
        except TemplateRefused as e:
            raise api.bad(str(e), "messages", "template_error")
        ids = _encode(st, text)
        p.media = None
        if images:
            try:
                ids, p.media = st.vision.prepare(ids, images)
            except MediaError as e:
                raise api.bad(str(e), "messages", e.code)
        return text, ids, note

    def split_tools(text, p):
        if not p.tools:
            return text, []
        if st.family:
            return st.fmt.split_tools(text, p.tools, p.tool_choice)
        return extract_tool_calls(text, st.fmt.tool_open, st.fmt.tool_close)

    async def render(request):
        try:
            body = await _json_body(request, st)
            p = api.parse_params(body, api.CHAT_FIELDS, st.defaults)
            with st.prep_gate:
                text, ids, note = render_chat(body, p)
            return JSONResponse({"prompt": text, "token_ids": ids, "count": len(ids)}, headers={"X-Rexl3-Note": note} if note else None)
        except api.ApiError as e:
            return _err(e)

    async def run(request, chat: bool):
        import time as _time
        t_in = _time.perf_counter()
        try:
            body = await _json_body(request, st)
            p = api.parse_params(body, api.CHAT_FIELDS if chat else api.COMPLETION_FIELDS, st.defaults)
            _check_model(st, p)
            _ready_or_503(st)
            note = None
            try:
                with st.prep_gate:
                    if chat:
                        prompt_text, ids, note = render_chat(body, p)
                    else:
                        pr = body.get("prompt")
                        if isinstance(pr, list) and pr and all(isinstance(t, int) and not isinstance(t, bool) for t in pr):
                            prompt_text, ids = "", list(pr)
                        elif isinstance(pr, str):
                            prompt_text, ids = pr, _encode(st, pr)
                        else:
                            raise api.bad("'prompt' must be a string or a list of token ids", "prompt")
            except budget.BudgetRefused as e:
                raise _budget_error(e)
            note_headers = {"X-Rexl3-Note": note} if note else None
            rid = api.new_id("chatcmpl" if chat else "cmpl")
            req = _make_request(st, ids, p, rid, prompt_text if chat else "")
            st.handle.metrics.observe("request_preprocessing_seconds", _time.perf_counter() - t_in)
            try:
                ticket = st.handle.submit(req, asyncio.get_running_loop())
            except OverflowError:
                raise api.ApiError(429, "the request queue is full", "rate_limit_error", "queue_full", retry_after=1)
            except RuntimeError as e:
                raise api.ApiError(503, f"engine is {e}", "service_unavailable", str(e), retry_after=5)
            reply = _Reply(st, p, chat, prompt_text)
            model = p.model or st.model_name
            if not p.stream:
                reason, usage = await _collect(st, ticket, reply)
                u = api.usage_object(usage, len(st.tok.encode(reply.reasoning)) if reply.reasoning else 0)
                if chat:
                    text, calls = split_tools(reply.text, p)
                    return JSONResponse(api.chat_completion(rid, model, text, reply.reasoning, calls, reason, u, st.fingerprint,
                                                            reply.ids if p.return_token_ids else None), headers=note_headers)
                return JSONResponse(api.text_completion(rid, model, reply.text, reason, u, st.fingerprint))

            async def gen():
                try:
                    if chat:
                        yield _sse(api.chat_chunk(rid, model, {"role": "assistant", "content": ""}, None, st.fingerprint))
                    while True:
                        try:
                            msg = await asyncio.wait_for(ticket.out.get(), timeout=15.0)
                        except asyncio.TimeoutError:
                            yield b": keep-alive\n\n"
                            continue
                        if msg[0] == "tokens":
                            c, r = reply.push(msg[1])
                            if chat:
                                if r:
                                    yield _sse(api.chat_chunk(rid, model, {"reasoning_content": r}, None, st.fingerprint))
                                if c:
                                    yield _sse(api.chat_chunk(rid, model, {"content": c}, None, st.fingerprint))
                            elif c:
                                yield _sse(api.text_completion(rid, model, c, None, None, st.fingerprint, stream_chunk=True))
                            if reply.stopped:
                                st.handle.cancel(ticket.id)
                        elif msg[0] == "done":
                            c, r = reply.finish()
                            reason = "stop" if reply.stopped else msg[1]
                            st.handle.metrics.inc("sse_terminal_total", kind=str(reason))
                            if chat:
                                if r:
                                    yield _sse(api.chat_chunk(rid, model, {"reasoning_content": r}, None, st.fingerprint))
                                if c:
                                    yield _sse(api.chat_chunk(rid, model, {"content": c}, None, st.fingerprint))
                                yield _sse(api.chat_chunk(rid, model, {}, api.finish_reason(reason), st.fingerprint))
                                if p.include_usage:
                                    yield _sse(api.chat_chunk(rid, model, {}, None, st.fingerprint, usage=api.usage_object(msg[2])))
                            else:
                                yield _sse(api.text_completion(rid, model, c, reason, api.usage_object(msg[2]) if p.include_usage else None,
                                                               st.fingerprint, stream_chunk=True))
                            break
                        else:
                            text = msg[2] if msg[0] == "refused" else str(msg[1])
                            yield _sse({"error": {"message": text, "type": "server_error", "code": msg[1] if msg[0] == "refused" else "engine_error",
                                                  "param": None}})
                            break
                    yield b"data: [DONE]\n\n"
                finally:
                    ticket.closed = True
                    st.handle.cancel(ticket.id)    # client gone (or done): free the slot

            return StreamingResponse(gen(), media_type="text/event-stream", headers={"Cache-Control": "no-cache", "X-Accel-Buffering": "no", **(note_headers or {})})
        except api.ApiError as e:
            return _err(e)

    async def chat(request):
        return await run(request, True)

    async def completions(request):
        return await run(request, False)

    routes = [Route("/health/live", live), Route("/health", health), Route("/health/ready", health), Route("/v1/health", health),
              Route("/v1/models", models), Route("/metrics", metrics), Route("/tokenize", tokenize, methods=["POST"]),
              Route("/v1/chat/completions", chat, methods=["POST"]), Route("/v1/completions", completions, methods=["POST"]),
              Route("/v1/chat/completions/render", render, methods=["POST"]), Route("/v1/decisions", decisions, methods=["POST"])]
    app = Starlette(routes=routes)
    app.state.rexl3 = st
    return _HttpMetrics(app, st.handle.metrics, {r.path for r in routes})


class _HttpMetrics:
    """ASGI wrapper: requests by route, responses by status code, and the time to the response headers.  Unknown paths count under one
    label so that a scanner cannot grow the label set."""

    def __init__(self, app, metrics, known_routes):
        self.app, self.metrics, self.known = app, metrics, known_routes
        self.state = app.state

    async def __call__(self, scope, receive, send):
        if scope["type"] != "http":
            await self.app(scope, receive, send)
            return
        import time as _time
        route = scope.get("path", "") if scope.get("path", "") in self.known else "other"
        t0 = _time.perf_counter()
        self.metrics.inc("http_requests_total", route=route)

        async def send_wrapped(message):
            if message["type"] == "http.response.start":
                code = str(message.get("status", 0))
                self.metrics.inc("http_responses_total", code=code)
                self.metrics.inc("http_route_responses_total", route=route, code=code)
                self.metrics.observe("http_headers_seconds", _time.perf_counter() - t0)
            await send(message)
        await self.app(scope, receive, send_wrapped)
