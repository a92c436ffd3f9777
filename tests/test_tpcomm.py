"""The TpComm collective interface: SingleRank, torch.distributed behind it (two gloo ranks on the CPU), and the peer-memory form over a loopback arena."""
import os
import subprocess
import sys
import threading

import pytest
import torch

from rexl3_b200.parallel import tpcomm

_GLOO = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["RX_ROOT"])
from rexl3_b200.parallel import tpcomm
dist.init_process_group("gloo", rank=int(os.environ["RANK"]), world_size=2)
c = tpcomm.NcclTp()
r = c.rank
buf = torch.arange(8, dtype=torch.float32) * (r + 1)
c.allreduce_sum_f32(buf)
assert torch.equal(buf, torch.arange(8, dtype=torch.float32) * 3)
out = torch.zeros(2, 4)
c.allgather_f32(torch.full((4,), float(r + 5)), out)
assert out.tolist() == [[5.0] * 4, [6.0] * 4]
recv = torch.zeros(4, dtype=torch.int32)
c.swap_bytes(torch.full((4,), r + 10, dtype=torch.int32), recv)
assert recv.tolist() == [11 - r] * 4
c.barrier()
assert c.capturable() is False and c.async_error() is None and c.aux() is c
dist.destroy_process_group()
print("TPCOMM_GLOO_OK", r)
'''


def test_single_rank_is_a_no_op():
    c = tpcomm.SingleRank()
    x = torch.arange(8, dtype=torch.float32)
    c.allreduce_sum_f32(x)
    out = torch.zeros(1, 8)
    c.allgather_f32(x, out)
    r = torch.zeros(8)
    c.swap_bytes(x, r)
    assert torch.equal(out[0], x) and torch.equal(r, x) and c.capturable() and c.async_error() is None


def test_torch_distributed_behind_the_interface(tmp_path):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "w.py"
    script.write_text(_GLOO)
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29577",
                                                                       RX_ROOT=root), stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=120)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs) and all("TPCOMM_GLOO_OK" in o for o in outs), outs


def test_layout_rejects_bad_capacities():
    with pytest.raises(ValueError):
        tpcomm.CollLayout(2, 6)
    L = tpcomm.CollLayout(4, 1024)
    assert L.total >= 4 * 2 * 4 * 1024 and L.slots % 256 == 0


@pytest.mark.gpu
@pytest.mark.parametrize("ranks", [2, 4])
def test_peer_memory_collectives_over_a_loopback_arena(ranks):
    """Every rank pushes into every rank's slot and sums locally in rank order: the same bits everywhere, equal to the serial rank-order sum;
    many collectives in a row reuse the two slot sets; all-gather and (two ranks) the byte swap."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    comms = tpcomm.loopback_group(ranks, 4096)
    g = torch.Generator(device="cuda").manual_seed(ranks)
    data = [torch.randn(12, 4096, device="cuda", generator=g) for _ in range(ranks)]
    results, errors = [None] * ranks, []

    def run(r):
        try:
            c = comms[r]
            sums = []
            for it in range(12):
                buf = data[r][it, :4096 - 4 * it].clone()
                c.allreduce_sum_f32(buf)
                sums.append(buf.clone())
            out = torch.zeros(ranks, 256, device="cuda")
            c.allgather_f32(data[r][0, :256].contiguous(), out)
            sw = None
            if ranks == 2:
                sw = torch.zeros(64, dtype=torch.int32, device="cuda")
                c.swap_bytes(torch.full((64,), r + 40, dtype=torch.int32, device="cuda"), sw)
            c.barrier()
            assert c.async_error() is None and not c.capturable()
            results[r] = (sums, out, sw)
        except Exception as e:          # noqa: BLE001
            errors.append((r, repr(e)))
            try:
                comms[r].host_barrier.abort()
            except Exception:           # noqa: BLE001
                pass

    threads = [threading.Thread(target=run, args=(r,)) for r in range(ranks)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(120)
    assert not errors, errors
    for it in range(12):
        want = data[0][it, :4096 - 4 * it].clone()
        for r in range(1, ranks):
            want = want + data[r][it, :4096 - 4 * it]          # rank order
        for r in range(ranks):
            assert torch.equal(results[r][0][it], want), (it, r)
    for r in range(ranks):
        assert torch.equal(results[r][1], torch.stack([data[q][0, :256] for q in range(ranks)]))
        if ranks == 2:
            assert results[r][2].tolist() == [41 - r] * 64
    comms[0].abort()
    with pytest.raises(tpcomm.TpCommError):
        comms[0].allreduce_sum_f32(torch.zeros(8, device="cuda"))
