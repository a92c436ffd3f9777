"""Guard bands around scratch buffers (the memory-checker stand-in)."""
import pytest
import torch

from rexl3_b200.utils import canary


def test_guard_bands_name_the_damaged_buffer():
    canary.forget()
    a = canary.guarded("t.a", (7, 5), torch.float32, "cpu", zero=True, force=True)
    b = canary.guarded("t.b", 33, torch.bfloat16, "cpu", force=True)
    assert a.shape == (7, 5) and a.dtype == torch.float32 and float(a.abs().sum()) == 0.0 and b.shape == (33,)
    a.fill_(3.0)
    b.fill_(1.0)
    assert canary.check_all() == 2
    whole = next(w for n, w, _ in canary._registry if n == "t.b")
    whole[canary.BAND_BYTES + 66 + 5] = 0          # a write 5 bytes past the end of b
    with pytest.raises(canary.CanaryError) as e:
        canary.check_all()
    assert "t.b" in str(e.value) and "after" in str(e.value) and "t.a" not in str(e.value)
    canary.forget("t.")
    assert canary.check_all() == 0


def test_off_by_default_is_a_plain_allocation(monkeypatch):
    monkeypatch.delenv("REXL3_CANARY", raising=False)
    canary.forget()
    x = canary.guarded("plain", (4, 4), torch.float16, "cpu")
    assert x.shape == (4, 4) and canary.check_all() == 0
