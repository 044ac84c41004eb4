"""Batch aggregation across caller threads (b200_mux_*): merged evaluations equal direct ones, requests are merged."""
import threading

import numpy as np
import pytest

from conftest import load_case
from lc0_b200 import _lib, network

pytestmark = pytest.mark.gpu


def test_requests_from_many_threads_are_merged_and_correct():
    net, pos, n, g = load_case("cfg3_mini")
    masks, values = np.array(pos["masks"]), np.array(pos["values"])
    nw = network.Network(net, "precision=fp32,max_batch=256")
    want = nw.evaluate(masks[:256], values[:256])
    mux = nw.new_mux(max_batch=256, wait_us=3000)
    errors = []

    def worker(k):
        try:
            rng = np.random.default_rng(k)
            for it in range(12):
                a = int(rng.integers(0, 200))
                cnt = int(rng.integers(1, 40))
                out = mux.evaluate(masks[a:a + cnt], values[a:a + cnt])
                bad = (np.abs(out["policy"] - want["policy"][a:a + cnt]).max() > 1e-5
                       or np.abs(out["q"] - want["q"][a:a + cnt]).max() > 1e-6
                       or np.abs(out["m"] - want["m"][a:a + cnt]).max() > 1e-5)
                if bad:
                    errors.append(("mismatch", k, it))
        except Exception as e:  # pragma: no cover
            errors.append(e)

    threads = [threading.Thread(target=worker, args=(k,)) for k in range(16)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors[:3]
    st = mux.stats()
    assert st["requests"] == 16 * 12
    assert st["batches"] < st["requests"] // 2  # with 16 callers in flight most launches carry several requests
    assert st["positions"] >= st["requests"]
    mux.close()
    assert nw.device_status() == 0
    nw.close()


def test_limits_and_errors():
    lib = _lib.load()
    net, pos, n, g = load_case("cfg3_mini")
    masks, values = np.array(pos["masks"]), np.array(pos["values"])
    nw = network.Network(net, "precision=fp32,max_batch=32")
    with pytest.raises(_lib.B200Error):
        nw.new_mux(max_batch=64)  # beyond the network's own limit
    mux = nw.new_mux(max_batch=16, wait_us=0)
    with pytest.raises(_lib.B200Error):
        mux.evaluate(masks[:17], values[:17])  # a request larger than the aggregator's batch
    out = mux.evaluate(masks[:16], values[:16])
    assert np.abs(out["q"] - g["q"][:16]).max() <= 1e-5
    assert mux.evaluate(masks[:0], values[:0])["q"].size == 0
    mux.close()
    nw.close()


def test_destroy_with_blocked_callers():
    """Destroying the aggregator while callers are inside it: every caller returns (with its result or with the
    'destroyed' error) and nothing touches freed memory: b200_mux_destroy waits until the last caller has left."""
    net, pos, n, g = load_case("cfg3_mini")
    masks, values = np.array(pos["masks"]), np.array(pos["values"])
    nw = network.Network(net, "precision=fp32,max_batch=64")
    for attempt in range(5):
        mux = nw.new_mux(max_batch=64, wait_us=200000)  # workers wait 0.2 s for more requests: callers stay blocked
        outcomes = []
        entering = [threading.Event() for _ in range(8)]

        def caller(k):
            try:
                entering[k].set()
                out = mux.evaluate(masks[k:k + 3], values[k:k + 3])
                outcomes.append(("ok", float(np.abs(out["q"] - g["q"][k:k + 3]).max())))
            except _lib.B200Error as e:
                outcomes.append(("error", str(e)))

        threads = [threading.Thread(target=caller, args=(k,)) for k in range(8)]
        for t in threads:
            t.start()
        import time
        for e in entering:
            e.wait()
        time.sleep(0.05 + 0.03 * attempt)  # every caller is inside b200_mux_eval by now, blocked on its request
        mux.close()
        for t in threads:
            t.join(timeout=30)
            assert not t.is_alive()
        assert len(outcomes) == 8
        for kind, val in outcomes:
            assert (kind == "ok" and val <= 1e-5) or (kind == "error" and "destroy" in val), (kind, val)
    nw.close()
