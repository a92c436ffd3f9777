"""The engine's exactness harness on the CUDA backend (real kernels, CUDA-graph replay)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def make_backend():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.engine.gpu_backend import DenseGpuBackend
    from rexl3_b200.models import dense
    cfg = dense.CONFIGS["test-hd128"]
    w = dense.random_weights(cfg, seed=3)
    model = dense.DenseGPU(w, num_pages=96, max_rows=64, max_seqs=8, max_blocks_per_seq=8, max_prefill_rows=512)
    state = {}

    def make():
        # one model, fresh bookkeeping (the KV pages are simply overwritten)
        state["b"] = DenseGpuBackend(model, max_slots=8)
        return state["b"]
    make.vocab = cfg.vocab
    return make


@pytest.mark.parametrize("check", ["row_invariance", "serial_batched_equals_solo", "drafted_equals_serial", "chunked_prefill_equals_whole",
                                   "rollback_equals_replay", "cached_equals_cold"])
def test_exactness_on_device(make_backend, check):
    from rexl3_b200.engine import harness
    assert getattr(harness, check)(make_backend, make_backend.vocab) is None


def test_smoke_entry():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import __graft_entry__ as g
    g.smoke()
