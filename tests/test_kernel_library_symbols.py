"""Every entry point the Python bindings declare exists in the built kernel library (a renamed or dropped launcher is caught on the CPU)."""
import ctypes
import re

from rexl3_b200.ops import lib


def test_every_declared_entry_point_is_exported():
    L = lib.load()
    src = open(lib.__file__).read()
    names = re.findall(r'^\s+"(rx_[a-z0-9_]+)":', src, flags=re.M)
    assert len(names) > 40
    missing = [n for n in names if not hasattr(L, n)]
    assert missing == []
    # and the bindings in kernels.py call nothing that is not declared
    import rexl3_b200.ops.kernels as K
    used = set(re.findall(r"L\.(rx_[a-z0-9_]+)\(", open(K.__file__).read()))
    assert used <= set(names), sorted(used - set(names))
    assert isinstance(L, ctypes.CDLL)
