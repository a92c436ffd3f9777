"""The commands the documentation shows name modules and flags that exist."""
import importlib
import importlib.util
import os
import re

HERE = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DOCS = [os.path.join(HERE, "README.md"), os.path.join(HERE, "docs", "SERVING.md")]


def test_documented_modules_import_and_server_flags_exist():
    from rexl3_b200.recipes import known_flags
    text = "\n".join(open(p).read() for p in DOCS)
    mods = set(re.findall(r"python -m (rexl3_b200(?:\.[a-z_0-9]+)*)", text)) | set(re.findall(r"-m (rexl3_b200\.server)\b", text))
    assert {"rexl3_b200.server", "rexl3_b200.quant", "rexl3_b200.plan", "rexl3_b200.release", "rexl3_b200.cluster", "rexl3_b200.router"} <= mods
    for m in sorted(mods):
        spec = importlib.util.find_spec(m)
        assert spec is not None, m
        if spec.submodule_search_locations is not None:       # a package: `python -m` needs its __main__
            assert importlib.util.find_spec(m + ".__main__") is not None, m
    flags = known_flags()
    for line in text.splitlines():
        if "rexl3_b200.server" in line and "python" in line:
            for f in re.findall(r"(--[a-z][a-z-]+)", line.split("rexl3_b200.server", 1)[1].split("#")[0]):
                assert f in flags, (f, line)
    # the option table of the serving guide
    serving = open(DOCS[1]).read()
    for f in re.findall(r"`(--[a-z][a-z-]+)", serving.split("| option | meaning |", 1)[1].split("## Several GPUs", 1)[0]):
        assert f in flags, f
