"""Lockstep control plane on CPU ranks (gloo, two processes): followers replay the leader's backend calls; a dropped message
is detected as a numbering gap.  No GPU is involved; failures are made on the host."""
import os
import socket

import pytest
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, drop, q):
    import datetime
    import torch.distributed as dist
    from rexl3_b200.engine import Engine, MockBackend, MockOptions, Request
    from rexl3_b200.engine.lockstep import GroupLost, LockstepLeader, follow
    from rexl3_b200.sampling import GREEDY
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    be = MockBackend(MockOptions(slots=4))
    try:
        if rank == 0:
            lead = LockstepLeader(be, dist.group.WORLD)
            eng = Engine(lead, None, window_rows=16, prefill_chunk=64, spec="copy")
            eng.submit(Request("a", list(range(1, 40)), 12, GREEDY))
            eng.submit(Request("b", list(range(5, 25)), 9, GREEDY))
            steps = 0
            while eng.has_work() and steps < 200:
                if drop and steps == 3:
                    lead.drop_next = True
                eng.step()
                steps += 1
            lead.stop()
            q.put((rank, "ok", lead.seq, sorted((s, len(c)) for s, c in be.ctx.items())))
        else:
            n = follow(be, dist.group.WORLD)
            q.put((rank, "ok", n + 1, sorted((s, len(c)) for s, c in be.ctx.items())))
    except GroupLost as e:
        q.put((rank, "lost", str(e), None))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def _run(drop):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_worker, args=(r, 2, port, drop, q)) for r in range(2)]
    for p in ps:
        p.start()
    out = {}
    for _ in ps:
        r = q.get(timeout=90)
        out[r[0]] = r[1:]
    for p in ps:
        p.join(timeout=30)
    return out


@pytest.mark.timeout(150)
def test_followers_replay_every_call():
    out = _run(False)
    assert out[0][0] == "ok" and out[1][0] == "ok", out
    assert out[0][1] == out[1][1]            # same number of calls (the stop included)
    assert out[0][2] == out[1][2]            # same slot state on both ranks


@pytest.mark.timeout(150)
def test_dropped_message_is_detected_as_a_gap():
    out = _run(True)
    assert out[1][0] == "lost" and "numbering gap" in out[1][1], out
