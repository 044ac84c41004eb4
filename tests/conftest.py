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


def load_compact(name):
    """(parsed net, positions npz, count, golden npz) of a large-batch golden: the golden holds `legal_logits`
    [count][256] (the reference's logits of each position's legal moves, zero padded) instead of all 1858."""
    from lc0_b200 import mknet, netproto
    g = np.load(os.path.join(GOLDEN, "golden_%s.npz" % name))
    pos = np.load(os.path.join(GOLDEN, "%s.npz" % str(g["positions"])))
    net_name = str(g["net"])
    if net_name not in _net_cache:
        _net_cache.clear()
        _net_cache[net_name] = netproto.parse_net(netproto.encode("Net", mknet.make_net(net_name)))
    return _net_cache[net_name], pos, int(g["count"]), g


def legal_logits(policy, pos, n):
    """[n][256] logits of the legal moves of the first n positions (zero padded), from full policy vectors."""
    legal = np.clip(np.asarray(pos["legal"][:n], np.int64), 0, 1857)
    out = np.take_along_axis(np.asarray(policy, np.float32), legal, axis=1)
    out[np.arange(256)[None, :] >= np.asarray(pos["n_legal"][:n])[:, None]] = 0
    return out


@pytest.fixture(scope="session")
def lib():
    from lc0_b200 import _lib
    return _lib.load()
