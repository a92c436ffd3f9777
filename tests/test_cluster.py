"""Cluster file validation, the supervisor's exit-code policy, and a supervised group of real (CPU) child processes."""
import json
import sys

import pytest

from rexl3_b200.cluster import Attempt, ClusterError, Policy, classify, supervise, validate
from rexl3_b200.cluster.schema import rank_commands
from rexl3_b200.cluster.supervise import LocalRunner

DOC = {"schema_version": 1, "name": "box", "nodes": [{"name": f"g{i}", "gpu": i} for i in range(4)], "random_init": "dense-27b",
       "serve": {"flags": ["--slots", "8"]}, "groups": [{"name": "a", "ranks": ["g0", "g1"], "tp_port": 29600, "http_port": 8080},
                                                         {"name": "b", "ranks": ["g2", "g3"], "tp_port": 29601, "http_port": 8081}]}


def test_validate_accepts_and_refuses():
    c = validate(DOC)
    assert list(c.groups) == ["a", "b"]
    cmds = rank_commands(c, "a")
    assert cmds[1][0]["RANK"] == "1" and cmds[1][0]["WORLD_SIZE"] == "2" and "--slots" in cmds[0][1]
    for bad in ({**DOC, "extra": 1}, {**DOC, "schema_version": 2},
                {**DOC, "groups": [{"name": "a", "ranks": ["g0", "gX"], "tp_port": 29600, "http_port": 8080}]},
                {**DOC, "groups": DOC["groups"] + [{"name": "c", "ranks": ["g0"], "tp_port": 29602, "http_port": 8082}]},
                {**DOC, "groups": [DOC["groups"][0], {**DOC["groups"][1], "http_port": 8080}]}):
        with pytest.raises(ClusterError):
            validate(json.loads(json.dumps(bad)))


def test_classify_exit_codes():
    assert classify(Attempt([0, 0], True)) == "clean"
    assert classify(Attempt([70, 70], True)) == "restart"
    assert classify(Attempt([101, None], True)) == "restart_once"
    assert classify(Attempt([1, None], False)) == "refusal"
    assert classify(Attempt([1, 70], True)) == "restart"
    assert classify(Attempt([2, None], True)) == "refusal"
    assert classify(Attempt([137, None], True)) == "restart"
    assert classify(Attempt([75, None], False)) == "restart"


def test_supervise_policy_restart_backoff_and_give_up():
    seq = [Attempt([70, 70], True, 5), Attempt([137, None], True, 5), Attempt([0, 0], True, 5)]
    slept = []
    assert supervise(lambda: seq.pop(0), Policy([1, 2, 4], 600, 5), sleep=slept.append, clock=lambda: 0.0, log=lambda s: None) == 0
    assert slept == [1, 2]
    seq = [Attempt([1, None], False), Attempt([1, None], False)]
    assert supervise(lambda: seq.pop(0), Policy(), sleep=lambda s: None, clock=lambda: 0.0, log=lambda s: None) == 78
    assert supervise(lambda: Attempt([70], True, 1), Policy([0], 600, 3), sleep=lambda s: None, clock=lambda: 0.0, log=lambda s: None) == 75


@pytest.mark.timeout(60)
def test_local_runner_restarts_the_whole_group():
    """Rank 1 of the first attempt exits 70 on its own; the runner tears rank 0 down; the second attempt ends cleanly."""
    import os
    import tempfile
    d = tempfile.mkdtemp()
    marker = os.path.join(d, "second")
    prog = ("import os,sys,time\n"
            f"m={marker!r}\n"
            "r=int(os.environ['RANK'])\n"
            "if os.path.exists(m): sys.exit(0)\n"
            "if r==1:\n time.sleep(2.0); open(m,'w').close(); sys.exit(70)\n"
            "time.sleep(30)\n")
    cmds = [({"RANK": str(r)}, [sys.executable, "-c", prog]) for r in range(2)]
    runs = []

    def attempt():
        a = LocalRunner(cmds)()
        runs.append(a.codes)
        return a
    assert supervise(attempt, Policy([0.0], 600, 5), log=lambda s: None) == 0
    assert runs[0][1] == 70 and runs[0][0] != 0 and runs[1] == [0, 0]


def test_single_rank_groups_pin_their_gpu_through_visibility():
    import json
    import os

    from rexl3_b200.cluster.schema import load_cluster, rank_commands
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    c = load_cluster(os.path.join(here, "docs", "examples", "cluster.b200-hybrid-dp8.json"))
    env, argv = rank_commands(c, "r5")[0]
    assert env["CUDA_VISIBLE_DEVICES"] == "5" and env["LOCAL_RANK"] == "0" and env["WORLD_SIZE"] == "1"
    assert argv[argv.index("--port") + 1] == "8085" and "gdn-hybrid-27b" in argv
    c8 = load_cluster(os.path.join(here, "docs", "examples", "cluster.b200-tp8.json"))
    envs = [e for e, _ in rank_commands(c8, "tp8")]
    assert all("CUDA_VISIBLE_DEVICES" not in e for e in envs) and [e["LOCAL_RANK"] for e in envs] == [str(i) for i in range(8)]
    assert json.dumps(envs[0])
