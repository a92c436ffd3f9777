import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

REFERENCE = os.environ.get("REXL3_REFERENCE_DIR", "")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    # the allocation-free entry point's test runs after every other test
    items.sort(key=lambda it: 1 if "test_zz_" in it.nodeid else 0)


@pytest.fixture(scope="session")
def reference_fixtures():
    p = os.path.join(REFERENCE, "testdata", "fixtures") if REFERENCE else ""
    if not p or not os.path.isdir(p):
        pytest.skip("set REXL3_REFERENCE_DIR to a reference checkout to run the conformance vectors")
    return p
