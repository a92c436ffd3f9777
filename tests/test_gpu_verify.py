"""Device verify / accept kernel against the host keyed sampler and accept rule."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_device_samples_and_accepts_like_the_host():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.ops import kernels as K
    from rexl3_b200.sampling import GREEDY, Sampling, choose
    from rexl3_b200.spec import accept
    rng = np.random.default_rng(0)
    count = 28
    specs = [(GREEDY, 100, 4), (Sampling(seed=7, temperature=0.8, top_k=20, top_p=0.9), 2000, 5), (Sampling(seed=99, temperature=1.3, top_k=0, top_p=1.0, min_p=0.05), 17, 1),
             (Sampling(seed=3, temperature=0.6, top_k=5, top_p=0.5), 123456, 3)]
    rows_ids, rows_vals, windows, host = [], [], [], []
    for s, pos, n in specs:
        ids = [np.sort(rng.choice(50000, size=count, replace=False)).astype(np.int32) for _ in range(n)]
        vals = [np.sort(rng.normal(0, 3, size=count).astype(np.float32))[::-1].copy() for _ in range(n)]
        samples = [choose(v, i, pos + j, s) for j, (v, i) in enumerate(zip(vals, ids))]
        # drafts: correct for the first two positions, then wrong
        drafts = [samples[j] if j < 2 else samples[j] + 1 for j in range(n - 1)]
        windows.append((s, pos, [11] + drafts))
        host.append((samples, accept(drafts, samples)))
        rows_ids += ids
        rows_vals += vals
    d_ids = torch.from_numpy(np.stack(rows_ids)).cuda()
    d_vals = torch.from_numpy(np.stack(rows_vals)).cuda()
    samples, accepted, err = K.verify_accept(d_ids, d_vals, windows)
    torch.cuda.synchronize()
    assert int(err[0]) == 0
    got = samples.cpu().tolist()
    r = 0
    for (hs, ha), a in zip(host, accepted.cpu().tolist()):
        assert got[r:r + len(hs)] == hs
        assert a == ha
        r += len(hs)


@pytest.mark.parametrize("bits", [2.0, 2.5, 4.0])
def test_cuda_trellis_encoder_matches_host_encoder(bits):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import time
    from rexl3_b200.format import exl3
    from rexl3_b200.quant import trellis
    b = exl3.Bits.of(bits)
    cb = "3inst" if b.is_integer else "mul1"
    rng = np.random.default_rng(int(bits * 10))
    tiles = rng.normal(0, 1.0, size=(6, 256)).astype(np.float32)
    want, werr = trellis.encode_tiles(tiles, b, cb)
    t0 = time.time()
    got, gerr = trellis.encode_tiles_cuda(tiles, b, cb)
    torch.cuda.synchronize()
    print(f"cuda encoder: {6 / (time.time() - t0):.1f} tiles/s at {bits} bpw")
    np.testing.assert_array_equal(got.cpu().numpy(), want)
    np.testing.assert_allclose(gerr.cpu().numpy(), werr, rtol=1e-6)


def test_quantize_linear_on_the_gpu_equals_the_host_quantizer():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.quant import quantize
    w = np.random.default_rng(4).normal(0, 0.02, size=(128, 256)).astype(np.float32)
    a = quantize.quantize_linear(w, 4.0, seed=3)
    b = quantize.quantize_linear(w, 4.0, seed=3, device="cuda")
    np.testing.assert_array_equal(a.trellis, b.trellis)
    np.testing.assert_array_equal(a.svh, b.svh)
