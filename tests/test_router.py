"""DP router: keying, sticky affinity, least-outstanding choice, health state machine, and the proxy end to end against
in-process mock backends (streaming pass-through, failover before the first byte, admin drain)."""
import asyncio
import json

import pytest

from rexl3_b200.router import AffinityMap, Backend, Fleet, affinity_key, fnv64, rendezvous


def test_keying_is_stable_and_prefix_based():
    assert fnv64(b"") == fnv64(b"") and fnv64(b"a") != fnv64(b"b")
    a = json.dumps({"messages": [{"role": "system", "content": "S"}, {"role": "user", "content": "hello"}, {"role": "assistant", "content": "x"},
                                 {"role": "user", "content": "more"}]}).encode()
    b = json.dumps({"messages": [{"role": "system", "content": "S"}, {"role": "user", "content": "hello"}]}).encode()
    ka, sa = affinity_key({}, a)
    kb, _ = affinity_key({}, b)
    assert ka == kb and sa == "prompt"                    # later turns of a conversation keep the key of turn one
    kh, sh = affinity_key({"x-affinity-key": "tenant-7"}, a)
    assert sh == "header" and kh == fnv64(b"tenant-7")
    assert affinity_key({}, b"not json") == (None, "none")
    assert rendezvous(5, 9) == rendezvous(5, 9)


def test_affinity_map_lru_and_ttl():
    now = [0.0]
    m = AffinityMap(cap=2, ttl_s=10, clock=lambda: now[0])
    m.put(1, "a"); m.put(2, "b"); m.put(3, "c")
    assert m.get(1) is None and m.evicted_capacity == 1
    now[0] = 11
    assert m.get(2) is None and m.evicted_ttl == 1


def test_choice_sticky_then_least_outstanding_and_health():
    f = Fleet([Backend("a", "http://a"), Backend("b", "http://b")], max_skew=2, fail_after=2, recover_after=2)
    first = f.choose(42)
    assert f.choose(42) is first                          # sticky
    first.inflight = 5                                    # overloaded past the skew: the key moves
    other = f.choose(42)
    assert other is not first and f.counters["sticky_moves"] == 1
    first.inflight = 0
    f.probe_result(other.name, False); assert other.healthy
    f.probe_result(other.name, False); assert not other.healthy
    assert f.choose(42) is first
    f.probe_result(other.name, True); assert not other.healthy
    f.probe_result(other.name, True); assert other.healthy
    f.set_admin("a", "draining"); f.set_admin("b", "disabled")
    assert f.choose(None) is None and not f.health()["ok"]


def test_proxy_end_to_end_with_failover_and_streaming():
    from aiohttp import web
    from aiohttp.test_utils import TestClient, TestServer
    from rexl3_b200.router.app import Router, build_apps

    async def run():
        hits = {"a": 0, "b": 0}

        def backend(name, broken=False):
            async def chat(request):
                hits[name] += 1
                if broken:
                    return web.json_response({"error": {"message": "engine unavailable"}}, status=503)
                r = web.StreamResponse(headers={"content-type": "text/event-stream"})
                await r.prepare(request)
                for i in range(3):
                    await r.write(f"data: {name}{i}\n\n".encode())
                await r.write_eof()
                return r

            async def ready(request):
                return web.Response(status=503 if broken else 200)
            app = web.Application()
            app.router.add_post("/v1/chat/completions", chat)
            app.router.add_get("/health/ready", ready)
            return app
        sa, sb = TestServer(backend("a", broken=True)), TestServer(backend("b"))
        await sa.start_server(); await sb.start_server()
        fleet = Fleet([Backend("a", str(sa.make_url("")).rstrip("/")), Backend("b", str(sb.make_url("")).rstrip("/"))])
        router = Router(fleet, probe_interval_s=3600)
        app, admin = build_apps(router)
        async with TestClient(TestServer(app)) as c, TestClient(TestServer(admin)) as ac:
            body = {"messages": [{"role": "user", "content": "hi"}], "stream": True}
            key, _ = affinity_key({}, json.dumps(body).encode())
            fleet.affinity.put(key, "a")                 # the conversation is pinned to the broken backend: the first request fails over
            for _ in range(3):
                r = await c.post("/v1/chat/completions", json=body)
                assert r.status == 200 and r.headers["x-rexl3-backend"] == "b"
                assert (await r.read()) == b"data: b0\n\ndata: b1\n\ndata: b2\n\n"          # byte-identical pass-through
            assert hits["a"] == 1 and fleet.counters["failovers"] == 1 and not fleet.backends["a"].healthy
            h = await c.get("/health")
            assert h.status == 200 and (await h.json())["ok"]
            r = await ac.post("/admin/backends", json={"op": "drain", "name": "b"})
            assert r.status == 200
            r = await c.post("/v1/chat/completions", json=body)
            assert r.status == 503
            m = await c.get("/metrics?scope=router")
            assert "rexl3_router_requests_total" in await m.text()
        await sa.close(); await sb.close()
    asyncio.run(run())
