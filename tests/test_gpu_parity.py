"""Parity of the CUDA path (through the C ABI) with the CPU oracle and the recorded reference outputs."""
import numpy as np
import pytest

from conftest import load_case
from lc0_b200 import _lib, mknet, network, weights
from oracle import oracle

pytestmark = pytest.mark.gpu

ALL = ["cfg1_mini", "cfg2_mini", "cfg3_mini", "cfg4_mini", "cfg1", "cfg2", "cfg3", "cfg4_2layer"]
# fp32 verification mode: error relative to the largest logit of the batch (north star: <= 1e-5).
FP32_REL = 1e-5
# fp16 storage with fp32 accumulation (north star: policy softmax and WDL/Q/M max-abs <= 2e-3).
HALF_ATOL = 2e-3


def _softmax_err_and_argmax(got, want, pos, n):
    worst, agree, decided = 0.0, 0, 0
    for i in range(n):
        lg = pos["legal"][i][:pos["n_legal"][i]]
        a = oracle.legal_softmax(got[i], lg)
        b = oracle.legal_softmax(want[i], lg)
        worst = max(worst, float(np.abs(a - b).max()))
        top = np.sort(b)[::-1]
        if len(top) < 2 or top[0] - top[1] > 2 * HALF_ATOL:  # near-ties may legitimately flip
            decided += 1
            agree += int(a.argmax() == b.argmax())
    return worst, agree, decided


@pytest.mark.parametrize("name", ALL)
def test_fp32_mode_matches_reference(name):
    net, pos, n, g = load_case(name)
    nw = network.Network(net, "precision=fp32,max_batch=%d" % n)
    out = nw.evaluate(pos["masks"][:n], pos["values"][:n])
    nw.close()
    scale = float(np.abs(g["policy"]).max())
    assert np.abs(out["policy"] - g["policy"]).max() <= FP32_REL * scale
    for k in ("q", "d", "m"):
        assert np.abs(out[k] - g[k]).max() <= FP32_REL * max(1.0, float(np.abs(g[k]).max()))
    worst, agree, decided = _softmax_err_and_argmax(out["policy"], g["policy"], pos, n)
    assert agree == decided


@pytest.mark.parametrize("tc", [True, False])
@pytest.mark.parametrize("name", ALL)
def test_fp16_mode_within_tolerance(name, tc):
    net, pos, n, g = load_case(name)
    nw = network.Network(net, "precision=fp16,max_batch=%d,tensor_cores=%d" % (n, int(tc)))
    out = nw.evaluate(pos["masks"][:n], pos["values"][:n])
    assert nw.device_status() == 0
    nw.close()
    worst, agree, decided = _softmax_err_and_argmax(out["policy"], g["policy"], pos, n)
    assert worst <= HALF_ATOL
    assert agree == decided
    assert np.abs(out["q"] - g["q"]).max() <= HALF_ATOL
    assert np.abs(out["d"] - g["d"]).max() <= HALF_ATOL
    assert np.all(np.abs(out["m"] - g["m"]) <= HALF_ATOL * np.maximum(1.0, np.abs(g["m"])))


@pytest.mark.parametrize("name", ["cfg3_mini", "cfg4_mini", "cfg4_2layer", "cfg2_mini"])
def test_bf16_mode_runs_close(name):
    """bf16 keeps 8 mantissa bits in the residual stream: looser bound, reported for completeness."""
    net, pos, n, g = load_case(name)
    nw = network.Network(net, "precision=bf16,max_batch=%d" % n)
    out = nw.evaluate(pos["masks"][:n], pos["values"][:n])
    nw.close()
    worst, agree, decided = _softmax_err_and_argmax(out["policy"], g["policy"], pos, n)
    assert worst <= HALF_ATOL
    assert np.abs(out["q"] - g["q"]).max() <= 1e-2


def test_full_bt4_class_net_fp16_against_reference():
    """The full 15-layer BT4-class network on the recorded reference outputs."""
    net, pos, n, g = load_case("cfg4")
    nw = network.Network(net, "precision=fp16,max_batch=%d" % n)
    out = nw.evaluate(pos["masks"][:n], pos["values"][:n])
    assert nw.device_status() == 0
    nw.close()
    worst, agree, decided = _softmax_err_and_argmax(out["policy"], g["policy"], pos, n)
    assert worst <= HALF_ATOL and agree == decided
    assert np.abs(out["q"] - g["q"]).max() <= HALF_ATOL
    assert np.abs(out["d"] - g["d"]).max() <= HALF_ATOL
    assert np.all(np.abs(out["m"] - g["m"]) <= HALF_ATOL * np.maximum(1.0, np.abs(g["m"])))


def test_computation_api_and_batch_shapes():
    """AddInput one by one, odd batch sizes, and independence of a sample from its batch neighbours."""
    net, pos, n, g = load_case("cfg4_mini")
    nw = network.Network(net, "precision=fp32,max_batch=40")
    ref = nw.evaluate(pos["masks"][:n], pos["values"][:n])
    for count in (1, 2, 3, 7, 31):
        c = nw.new_computation()
        for i in range(count):
            c.add_input(pos["masks"][i], pos["values"][i])
        assert c.get_batch_size() == count
        c.compute_blocking()
        for i in range(count):
            np.testing.assert_allclose(c.policy(i), ref["policy"][i], atol=2e-6)
            assert abs(c.get_q_val(i) - ref["q"][i]) < 2e-6
            assert abs(c.get_d_val(i) - ref["d"][i]) < 2e-6
            assert abs(c.get_m_val(i) - ref["m"][i]) < 2e-6
            assert c.get_p_val(i, 5) == c.policy(i)[5]
        c.close()
    empty = nw.new_computation()
    empty.compute_blocking()
    assert empty.get_batch_size() == 0
    c = nw.new_computation()
    c.add_inputs(pos["masks"][:32], pos["values"][:32])
    with pytest.raises(_lib.B200Error, match="max_batch"):
        c.add_inputs(pos["masks"][:32], pos["values"][:32])
    nw.close()


def test_mlh_option_and_head_errors():
    net, pos, n, g = load_case("cfg3_mini")
    nw = network.Network(net, "precision=fp32,max_batch=8,mlh=false")
    out = nw.evaluate(pos["masks"][:4], pos["values"][:4])
    assert np.all(out["m"] == 0) and nw.get_capabilities()["moves_left"] == 0
    nw.close()
    with pytest.raises(weights.WeightsError):
        network.Network(net, "policy_head=optimistic")
    with pytest.raises(_lib.B200Error, match="Invalid GPU Id"):
        network.Network(net, "gpu=99")


def test_large_batch_consistency():
    """Batch 1024 in fp16 equals the same positions evaluated in chunks (tile tails, many CTAs per GEMM)."""
    net, pos, n, g = load_case("cfg4_mini")
    nw = network.Network(net, "precision=fp16,max_batch=1024")
    masks, values = pos["masks"], pos["values"]
    big = nw.evaluate(masks, values)
    small = nw.evaluate(masks[:100], values[:100])
    assert nw.device_status() == 0
    nw.close()
    np.testing.assert_allclose(big["policy"][:100], small["policy"], atol=1e-6)
    np.testing.assert_allclose(big["q"][:100], small["q"], atol=1e-6)


def test_graph_replay_matches_plain_launches():
    """The captured CUDA graph (third and later calls of a shape) gives the same numbers as plain launches."""
    net, pos, n, g = load_case("cfg4_mini")
    plain = network.Network(net, "precision=fp16,max_batch=32,graph_capture=0")
    want = plain.evaluate(pos["masks"][:n], pos["values"][:n])
    plain.close()
    nw = network.Network(net, "precision=fp16,max_batch=32")
    for i in range(4):  # plain, capture + replay, replay, replay
        got = nw.evaluate(pos["masks"][:n], pos["values"][:n])
        np.testing.assert_array_equal(got["policy"], want["policy"])
        np.testing.assert_array_equal(got["q"], want["q"])
    # a different batch size gets its own graph (tiny batches route some products to the FMA kernel, hence atol)
    for i in range(3):
        other = nw.evaluate(pos["masks"][:5], pos["values"][:5])
        np.testing.assert_allclose(other["policy"], want["policy"][:5], atol=HALF_ATOL)
    count = nw.launch_count()
    nw.evaluate(pos["masks"][:n], pos["values"][:n])
    assert nw.launch_count() > count  # replays are still counted as kernel launches
    assert nw.device_status() == 0
    nw.close()


def test_computation_may_outlive_its_network():
    """A garbage-collected host may destroy the network before its computations: results stay readable."""
    net, pos, n, g = load_case("cfg3_mini")
    nw = network.Network(net, "precision=fp32,max_batch=8")
    comps = []
    for i in range(3):
        c = nw.new_computation()
        c.add_inputs(pos["masks"][:4], pos["values"][:4])
        c.compute_blocking()
        comps.append(c)
    want = comps[0].policy(2)
    nw.close()
    for c in comps:
        np.testing.assert_array_equal(c.policy(2), want)
        assert abs(c.get_q_val(1) - g["q"][1]) < 1e-5
        c.close()


def test_concurrent_computations_on_two_slots():
    """Two host threads drive their own computations at the same time (lc0 runs several search threads)."""
    import threading
    net, pos, n, g = load_case("cfg4_mini")
    nw = network.Network(net, "precision=fp16,max_batch=32,slots=2")
    masks, values = np.array(pos["masks"]), np.array(pos["values"])  # the lazy .npz reader is not thread-safe
    want = nw.evaluate(masks[:n], values[:n])
    errors = []

    def worker(offset):
        try:
            for it in range(12):
                count = 5 + (it + offset) % 20
                c = nw.new_computation()
                c.add_inputs(masks[:count], values[:count])
                c.compute_blocking()
                got = np.stack([c.policy(i) for i in range(count)])
                if np.abs(got - want["policy"][:count]).max() > HALF_ATOL:
                    errors.append(("mismatch", offset, it))
                c.close()
        except Exception as e:  # pragma: no cover
            errors.append(e)

    threads = [threading.Thread(target=worker, args=(k,)) for k in range(3)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    assert nw.device_status() == 0
    nw.close()


def test_merged_qkv_and_smolgen_compression_launch_matches_separate_launches():
    """Q, K, V and the smolgen compression computed by one launch of the CTA-pair kernel (second output, narrow last
    tile) against the same network with the compression as a product of its own."""
    net = mknet.make_net("cfg4_2layer")
    rng = np.random.default_rng(5)
    n = 64
    masks = rng.integers(0, 2 ** 63, size=(n, 112), dtype=np.int64).astype(np.uint64) & rng.integers(
        0, 2 ** 63, size=(n, 112), dtype=np.int64).astype(np.uint64)
    values = np.ones((n, 112), np.float32)
    outs = []
    for flag in ("1", "0"):
        nw = network.Network(net, "precision=fp16,max_batch=%d,merge_compress=%s" % (n, flag))
        outs.append(nw.evaluate(masks, values))
        assert nw.device_status() == 0
        nw.close()
    scale = np.abs(outs[1]["policy"]).max()
    assert np.abs(outs[0]["policy"] - outs[1]["policy"]).max() <= 2e-3 * scale
    assert np.abs(outs[0]["q"] - outs[1]["q"]).max() <= 2e-3


def test_split_last_wave_matches_whole_tiles():
    """Products whose last wave of 256x256 tiles fills at most half of the CTA pairs compute that wave as half-width
    tiles (out-projection and FFN2 here, both with residual input and row statistics): same results as whole tiles."""
    net = mknet.make_net("cfg4_2layer")
    rng = np.random.default_rng(17)
    n = 96  # 96 tiles per 1024-wide product on 74 pairs: 22 tiles in the last wave
    masks = rng.integers(0, 2 ** 63, size=(n, 112), dtype=np.int64).astype(np.uint64) & rng.integers(
        0, 2 ** 63, size=(n, 112), dtype=np.int64).astype(np.uint64)
    values = np.ones((n, 112), np.float32)
    outs = []
    for flag in ("1", "0"):
        nw = network.Network(net, "precision=fp16,max_batch=%d,split_last_wave=%s" % (n, flag))
        outs.append(nw.evaluate(masks, values))
        assert nw.device_status() == 0
        nw.close()
    # the same MMAs on the same operands, in a different order over the CTA pairs: identical up to the atomics'
    # summation order in the row statistics
    scale = np.abs(outs[1]["policy"]).max()
    assert np.abs(outs[0]["policy"] - outs[1]["policy"]).max() <= 1e-3 * scale
    assert np.abs(outs[0]["q"] - outs[1]["q"]).max() <= 1e-3
