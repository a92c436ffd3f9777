"""Tensor parallelism across real GPUs (one process per GPU, fused peer-memory kernels, lockstep followers).  Needs at
least two GPUs (the one-rank case runs the same kernels and leader code on one GPU); NVLS is switched off for the children (only the CPU control group and plain peer stores are used)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("ranks", [1, 2, 4])
def test_tp_selftest_over_gpus(ranks):
    if not torch.cuda.is_available() or torch.cuda.device_count() < ranks:
        pytest.skip(f"needs {ranks} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}", "--master-addr", "127.0.0.1",
           "--master-port", str(29540 + ranks), "-m", "rexl3_b200.parallel.selftest"]
    r = subprocess.run(cmd, cwd=root, env=env, capture_output=True, text=True, timeout=420)
    assert r.returncode == 0 and f"TP_SELFTEST_OK ranks={ranks}" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_lost_rank_is_detected_without_a_hang():
    """A follower leaves between two steps (stream drained, nothing in flight); the leader notices on the host or through the bounded
    peer waits of its next step, within seconds.  NVLS off, plain peer stores only."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29549",
           "-m", "rexl3_b200.parallel.selftest", "--leave-after", "12"]
    r = subprocess.run(cmd, cwd=root, env=env, capture_output=True, text=True, timeout=240)
    assert "TP_FAILURE_DETECTED" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


def test_tp_windows_above_the_packet_size_with_the_in_switch_sum():
    """24 concurrent streams: the decode windows are wider than the packet format, so the ranks exchange f32 rows; where the fabric
    offers NVLink multicast the sum comes from `multimem.ld_reduce` (the self test prints which form ran).  Every rank stays alive to
    the end, so NVLS may be on here (the failure test above keeps it off)."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29551",
           "-m", "rexl3_b200.parallel.selftest", "--streams", "24"]
    r = subprocess.run(cmd, cwd=root, env=env, capture_output=True, text=True, timeout=420)
    assert r.returncode == 0 and "TP_SELFTEST_OK ranks=2" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_tree_rounds_over_a_tensor_parallel_group():
    """Verify windows of draft trees on 2 ranks: the tree arrays and the accepted paths' row copies reach every rank, tokens equal the chain-free run's."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 CUDA devices")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29553",
           "-m", "rexl3_b200.parallel.selftest", "--trees"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "TP_SELFTEST_OK" in r.stdout and "tp selftest trees" in r.stdout, r.stdout[-1500:] + r.stderr[-3000:]


@pytest.mark.parametrize("ranks", [2, 4])
def test_token_all_to_all_over_gpus_equals_one_gpu(ranks):
    """Data-parallel rows + token all-to-all over NVLink peer memory, one process per GPU: every rank's logits on its own sequence equal
    the one-GPU executor's bit for bit (prefill and decode steps)."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < ranks:
        pytest.skip(f"needs {ranks} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}", "--master-addr", "127.0.0.1",
           "--master-port", str(29560 + ranks), "-m", "rexl3_b200.parallel.a2a_selftest", "--skip-timing"]
    r = subprocess.run(cmd, cwd=root, env=env, capture_output=True, text=True, timeout=420)
    assert r.returncode == 0 and '"bitwise_equal_to_one_gpu": true' in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_tpcomm_peer_memory_collectives_over_gpus():
    """The generic collective interface on two real GPUs: the peer-memory all-reduce equals the serial rank-order sum bit for bit and the
    all-gather equals NCCL's (the self test also times both)."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29571",
           "-m", "rexl3_b200.parallel.tpcomm_selftest"]
    r = subprocess.run(cmd, cwd=root, env=env, capture_output=True, text=True, timeout=420)
    assert r.returncode == 0 and '"equal_to_rank_order_sum": true' in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
