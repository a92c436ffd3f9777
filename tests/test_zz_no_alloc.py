"""The allocation-free top-k entry point, called through its exported C symbol.

For callers that cannot allocate device memory (sealed memory plan, foreign stream callback): the scratch lives in a
fixed array inside the library.  Checked against the ordinary entry point on two calls in a row (the array is shared
and keeps the previous call's contents), and that sizes beyond the fixed array are refused.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_topk_matches_the_allocating_entry_point_twice():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.ops import kernels as K, lib
    L = ctypes.CDLL(lib.LIB_PATH)
    fn = L.rx_topk_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    stream = torch.cuda.current_stream().cuda_stream
    for trial, (rows, vocab, count) in enumerate([(5, 151936, 28), (64, 32000, 64)]):
        torch.manual_seed(trial)
        logits = torch.randn(rows, vocab, device="cuda")
        logits[0, 3] = logits[0, vocab - 1] = 50.0          # a tie: the lower id comes first
        ids = torch.full((rows, count), -1, dtype=torch.int32, device="cuda")
        vals = torch.zeros(rows, count, dtype=torch.float32, device="cuda")
        assert fn(logits.data_ptr(), rows, vocab, count, ids.data_ptr(), vals.data_ptr(), stream) == 0
        ref_ids = torch.empty_like(ids)
        ref_vals = torch.empty_like(vals)
        K.topk(logits, count, K.topk_scratch(rows, vocab, count), ref_ids, ref_vals)
        torch.cuda.synchronize()
        assert torch.equal(ids, ref_ids) and torch.equal(vals, ref_vals)
        assert ids[0, 0].item() == 3 and ids[0, 1].item() == vocab - 1
    small = torch.randn(65, 1000, device="cuda")
    out_i = torch.empty(65, 4, dtype=torch.int32, device="cuda")
    out_v = torch.empty(65, 4, dtype=torch.float32, device="cuda")
    assert fn(small.data_ptr(), 65, 1000, 4, out_i.data_ptr(), out_v.data_ptr(), stream) == 1      # too many rows
    assert fn(small.data_ptr(), 4, 300000, 4, out_i.data_ptr(), out_v.data_ptr(), stream) == 1     # vocabulary too large
    assert fn(small.data_ptr(), 4, 1000, 65, out_i.data_ptr(), out_v.data_ptr(), stream) == 1      # too many candidates
    torch.cuda.synchronize()
