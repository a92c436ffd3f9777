"""The router's HTTP side (aiohttp): streaming pass-through, one-shot failover before the first byte, health prober, admin
listener, metrics.  A reply forwarded through the router is byte-identical to the backend's own.
Behaviour parity: reference crates/router/src/handlers.rs, admin.rs, main.rs:14-43.

    python -m rexl3_b200.router --endpoint a=http://127.0.0.1:8001 --endpoint b=http://127.0.0.1:8002 --port 8000
"""
from __future__ import annotations

import argparse
import asyncio
import json
import sys

import aiohttp
from aiohttp import web

from .core import AffinityMap, Backend, Fleet
from .keying import affinity_key

HOP = {"connection", "keep-alive", "proxy-authenticate", "proxy-authorization", "te", "trailers", "transfer-encoding", "upgrade", "host", "content-length"}


def _is_engine_unavailable(status: int, body: bytes) -> bool:
    return status == 503 and (b"engine" in body.lower() or b"unavailable" in body.lower() or not body)


class Router:
    def __init__(self, fleet: Fleet, replay_cap: int = 8 << 20, probe_interval_s: float = 1.0, connect_timeout_s: float = 3.0, admin_token: str = ""):
        self.fleet, self.replay_cap, self.probe_interval, self.admin_token = fleet, replay_cap, probe_interval_s, admin_token
        self.timeout = aiohttp.ClientTimeout(total=None, connect=connect_timeout_s, sock_connect=connect_timeout_s)
        self.session: aiohttp.ClientSession | None = None
        self._prober = None

    # ---- lifecycle
    async def start(self, app=None):
        self.session = aiohttp.ClientSession(timeout=self.timeout, auto_decompress=False)
        self._prober = asyncio.create_task(self._probe_loop())

    async def stop(self, app=None):
        if self._prober:
            self._prober.cancel()
        if self.session:
            await self.session.close()

    async def probe_once(self):
        async def one(b: Backend):
            try:
                async with self.session.get(b.url + "/health/ready", timeout=aiohttp.ClientTimeout(total=2.0)) as r:
                    self.fleet.probe_result(b.name, r.status == 200)
            except Exception:
                self.fleet.probe_result(b.name, False)
        await asyncio.gather(*(one(b) for b in list(self.fleet.backends.values())))

    async def _probe_loop(self):
        while True:
            await self.probe_once()
            await asyncio.sleep(self.probe_interval)

    # ---- data path
    async def proxy(self, request: web.Request) -> web.StreamResponse:
        body = await request.read()
        key, _src = affinity_key(request.headers, body) if request.method == "POST" else (None, "none")
        headers = {k: v for k, v in request.headers.items() if k.lower() not in HOP}
        tried = []
        for attempt in range(2):
            b = self.fleet.choose(key, exclude=tried)
            if b is None:
                return web.json_response({"error": {"message": "no routable backend", "type": "router_unavailable"}}, status=503)
            tried.append(b.name)
            self.fleet.begin(b)
            ok = False
            try:
                try:
                    resp = await self.session.request(request.method, b.url + request.rel_url.raw_path_qs, data=body or None, headers=headers)
                except (aiohttp.ClientConnectorError, asyncio.TimeoutError, aiohttp.ServerDisconnectedError):
                    self.fleet.data_path_down(b.name)
                    if attempt == 0 and len(body) <= self.replay_cap:
                        self.fleet.counters["failovers"] += 1
                        continue
                    return web.json_response({"error": {"message": f"backend {b.name} unreachable", "type": "bad_gateway"}}, status=502)
                async with resp:
                    if resp.status == 503:
                        payload = await resp.read()
                        if _is_engine_unavailable(resp.status, payload):
                            self.fleet.data_path_down(b.name)
                            if attempt == 0 and len(body) <= self.replay_cap:
                                self.fleet.counters["failovers"] += 1
                                continue
                        return web.Response(status=503, body=payload, headers={k: v for k, v in resp.headers.items() if k.lower() not in HOP})
                    out = web.StreamResponse(status=resp.status, headers={k: v for k, v in resp.headers.items() if k.lower() not in HOP})
                    out.headers["x-rexl3-backend"] = b.name
                    await out.prepare(request)
                    try:
                        async for chunk in resp.content.iter_any():      # after the first byte nothing is retried
                            await out.write(chunk)
                        await out.write_eof()
                        ok = True
                    except (aiohttp.ClientError, ConnectionResetError, asyncio.CancelledError):
                        pass                                             # a dying stream reaches the client as a broken stream
                    return out
            finally:
                self.fleet.end(b, ok)
        return web.json_response({"error": {"message": "no backend accepted the request", "type": "bad_gateway"}}, status=502)

    async def health(self, request):
        h = self.fleet.health()
        return web.json_response(h, status=200 if h["ok"] else 503)

    async def metrics(self, request):
        f = self.fleet
        lines = [f"rexl3_router_{k}_total {v}" for k, v in f.counters.items()]
        lines.append(f"rexl3_router_affinity_entries {len(f.affinity)}")
        for b in f.backends.values():
            lab = f'{{backend="{b.name}"}}'
            lines += [f"rexl3_router_backend_inflight{lab} {b.inflight}", f"rexl3_router_backend_routable{lab} {int(b.routable)}",
                      f"rexl3_router_backend_served_total{lab} {b.served}", f"rexl3_router_backend_failed_total{lab} {b.failed}"]
        if request.query.get("scope") != "router":
            for b in list(f.backends.values()):
                try:
                    async with self.session.get(b.url + "/metrics", timeout=aiohttp.ClientTimeout(total=2.0)) as r:
                        for ln in (await r.text()).splitlines():
                            if ln.startswith("rexl3_") and not ln.startswith("rexl3_router_"):
                                name, _, rest = ln.partition(" ")
                                base, brace, labels = name.partition("{")
                                labels = f'backend="{b.name}"' + ("," + labels.rstrip("}") if brace else "")
                                lines.append(f"rexl3_router_{base[len('rexl3_'):]}{{{labels}}} {rest}")
                except Exception:
                    pass
        return web.Response(text="\n".join(lines) + "\n", content_type="text/plain")

    # ---- admin
    def _authorized(self, request) -> bool:
        return not self.admin_token or request.headers.get("authorization") == f"Bearer {self.admin_token}"

    async def admin(self, request: web.Request):
        if not self._authorized(request):
            return web.json_response({"error": "unauthorized"}, status=401)
        f = self.fleet
        if request.method == "GET":
            return web.json_response(f.health())
        try:
            doc = await request.json()
            op, name = doc.get("op"), doc.get("name")
            if op == "add":
                f.add(name, doc["url"])
            elif op == "remove":
                f.remove(name)
            elif op in ("drain", "disable", "enable"):
                f.set_admin(name, {"drain": "draining", "disable": "disabled", "enable": "enabled"}[op])
            else:
                return web.json_response({"error": f"unknown op {op!r}"}, status=400)
        except (KeyError, ValueError, json.JSONDecodeError) as e:
            return web.json_response({"error": str(e)}, status=400)
        return web.json_response(f.health())


def build_apps(router: Router):
    app = web.Application(client_max_size=256 << 20)
    app.on_startup.append(router.start)
    app.on_cleanup.append(router.stop)
    app.router.add_get("/health", router.health)
    app.router.add_get("/metrics", router.metrics)
    app.router.add_route("*", "/{tail:.*}", router.proxy)
    admin = web.Application()
    admin.router.add_route("*", "/admin/backends", router.admin)
    return app, admin


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="rexl3-router", allow_abbrev=False)
    p.add_argument("--endpoint", action="append", default=[], help="NAME=URL or URL (repeatable)")
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=8000)
    p.add_argument("--admin-bind", default="", help="HOST:PORT of the admin listener (off when empty)")
    p.add_argument("--admin-token", default="")
    p.add_argument("--affinity-max-skew", type=int, default=8)
    p.add_argument("--affinity-cap", type=int, default=65536)
    p.add_argument("--affinity-ttl-s", type=float, default=1800)
    p.add_argument("--probe-interval-ms", type=int, default=1000)
    p.add_argument("--probe-fail-after", type=int, default=3)
    p.add_argument("--probe-recover-after", type=int, default=2)
    p.add_argument("--replay-body-cap-bytes", type=int, default=8 << 20)
    a = p.parse_args(argv)
    if not a.endpoint:
        p.error("at least one --endpoint is required")
    backends = []
    for i, e in enumerate(a.endpoint):
        name, sep, url = e.partition("=")
        if not sep or name.startswith("http"):
            name, url = f"b{i}", e
        backends.append(Backend(name, url.rstrip("/")))
    fleet = Fleet(backends, a.affinity_max_skew, a.probe_fail_after, a.probe_recover_after, AffinityMap(a.affinity_cap, a.affinity_ttl_s))
    router = Router(fleet, a.replay_body_cap_bytes, a.probe_interval_ms / 1e3, admin_token=a.admin_token)
    app, admin = build_apps(router)

    async def run():
        runner = web.AppRunner(app)
        await runner.setup()
        await web.TCPSite(runner, a.host, a.port).start()
        if a.admin_bind:
            ah, _, ap_ = a.admin_bind.rpartition(":")
            ar = web.AppRunner(admin)
            await ar.setup()
            await web.TCPSite(ar, ah or "127.0.0.1", int(ap_)).start()
        print(f"rexl3-router event=start port={a.port} backends={len(backends)}", file=sys.stderr, flush=True)
        while True:
            await asyncio.sleep(3600)
    try:
        asyncio.run(run())
    except KeyboardInterrupt:
        pass
    return 0
