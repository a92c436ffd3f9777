"""Shard proofs: the planner mirror equals the library's planner; verdicts per cut; on a GPU a column slice keeps the whole matrix's bits."""
import pytest
import torch

from rexl3_b200.parallel import shard_proof as sp


def test_planner_mirror_equals_the_library():
    from rexl3_b200.ops import kernels as K
    for k in (256, 1024, 5120, 17408):
        for n in (128, 1024, 5120, 34816, 151936 // 128 * 128):
            for dec in (True, False):
                assert sp.plan_splits(k, n, dec) == K.plan_splits(k, n, dec), (k, n, dec)


def test_proof_table_verdicts():
    from rexl3_b200.models import dense
    cfg = dense.CONFIGS["dense-27b"]
    for ranks in (2, 4, 8):
        t = {p.name: p for p in sp.proof_table(sp.dense_shapes(cfg), ranks)}
        assert t["o"].verdict == "rank_order" and t["down"].verdict == "rank_order"
        for name in ("qkv", "gate_up", "lm_head"):
            p = t[name]
            assert p.verdict == ("same_plan" if p.local_splits == p.whole_splits else "pinned")
            assert p.local[1] * ranks >= p.N and p.local[1] % 128 == 0
    # a narrow matrix gets more K splits when it is cut: the shard must pin the whole matrix's count
    t = {p.name: p for p in sp.proof_table(dict(m=(4096, 8192, "columns")), 8)}
    assert t["m"].verdict == "pinned" and t["m"].local_splits > t["m"].whole_splits
    assert sp.main(["--config", "dense-27b", "--ranks", "2"]) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("bits", [4.0, 3.0])
def test_column_slices_keep_the_bits_on_the_device(bits):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import numpy as np
    from rexl3_b200.models.dense import random_linear
    from rexl3_b200.ops import kernels as K
    l = random_linear(1024, 1536, bits, np.random.default_rng(3), "3inst", 0.03)
    w = K.Exl3Weight.from_numpy(l.trellis, l.suh, l.svh, None, l.codebook, "cuda")
    for ranks in (2, 4):
        assert all(sp.compare_slices(w, ranks).values()), ranks
