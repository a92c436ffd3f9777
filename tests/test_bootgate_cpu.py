"""The tensor-parallel boot gate over a gloo group of two CPU ranks: agreeing ranks pass, a rank with another flag fails on both."""
import os
import subprocess
import sys
import textwrap

from rexl3_b200.models import dense
from rexl3_b200.parallel import bootgate


def test_collect_and_compare(tmp_path):
    lib = tmp_path / "k.so"
    lib.write_bytes(b"abc")
    cfg = dense.CONFIGS["tiny-llama"]
    a = bootgate.collect_facts(cfg, world=2, flags={"slots": 4, "graphs": True}, libraries=[str(lib)])
    b = bootgate.collect_facts(cfg, world=2, flags={"slots": 8, "graphs": True}, libraries=[str(lib), str(tmp_path / "none.so")])
    assert a["model"] == "tiny-llama" and len(a["config"]) == 16 and a["lib:k.so"] == bootgate.file_sha256(str(lib))[:16]
    assert bootgate.compare([a, dict(a)]) == []
    diffs = bootgate.compare([a, b])
    assert any("flag:slots = 8" in d for d in diffs) and any("lib:none.so = 'missing'" in d for d in diffs) and len(diffs) == 2


RANK = textwrap.dedent("""
    import os, sys, datetime
    import torch.distributed as dist
    from rexl3_b200.models import dense
    from rexl3_b200.parallel import bootgate
    rank = int(os.environ["RANK"])
    dist.init_process_group("gloo", rank=rank, world_size=2, timeout=datetime.timedelta(seconds=60))
    slots = 4 if (rank == 0 or sys.argv[1] == "same") else 8
    facts = bootgate.collect_facts(dense.CONFIGS["tiny-llama"], world=2, flags={"slots": slots}, libraries=[])
    try:
        got = bootgate.gate(facts)
        print("PASS", len(got))
    except bootgate.BootGateError as e:
        print("REFUSED", "flag:slots" in str(e))
    dist.destroy_process_group()
""")


def _run(mode, port):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, "-c", RANK, mode], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE, text=True) for r in range(2)]
    return [p.communicate(timeout=120)[0].strip().splitlines()[-1] for p in procs]


def test_gate_passes_when_ranks_agree_and_refuses_on_every_rank_when_not():
    assert _run("same", 29731) == ["PASS 2", "PASS 2"]
    assert _run("differ", 29732) == ["REFUSED True", "REFUSED True"]
