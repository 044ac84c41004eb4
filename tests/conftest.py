import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


_net_cache = {}


def load_case(name):
    """(parsed net, positions npz, count, golden npz) of a seeded synthetic network."""
    from lc0_b200 import mknet, netproto
    g = np.load(os.path.join(GOLDEN, "golden_%s.npz" % name))
    pos = np.load(os.path.join(GOLDEN, "%s.npz" % str(g["positions"])))
    if name not in _net_cache:
        _net_cache.clear()  # one big net at a time
        _net_cache[name] = netproto.parse_net(netproto.encode("Net", mknet.make_net(name)))
    return _net_cache[name], pos, int(g["count"]), g


@pytest.fixture(scope="session")
def lib():
    from lc0_b200 import _lib
    return _lib.load()
