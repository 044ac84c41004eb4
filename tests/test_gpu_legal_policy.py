"""Device-side legal-move softmax (the caller-side SoftmaxPolicy of lc0's wrapper moved behind the C ABI)."""
import numpy as np
import pytest

from conftest import load_case
from lc0_b200 import _lib, network
from oracle import oracle

pytestmark = pytest.mark.gpu


def _run(nw, pos, n, temperature=1.0, compact=False):
    c = nw.new_computation()
    c.set_policy_options(temperature=temperature, compact=compact)
    for i in range(n):
        c.add_input_with_moves(pos["masks"][i], pos["values"][i], pos["legal"][i][:pos["n_legal"][i]])
    c.compute_blocking()
    return c


@pytest.mark.parametrize("name", ["cfg4_mini", "cfg1_mini"])
def test_matches_host_formula_bit_exactly_and_reference_closely(name):
    net, pos, n, g = load_case(name)
    nw = network.Network(net, "precision=fp32,max_batch=%d" % n)
    c = _run(nw, pos, n)
    for i in range(n):
        ids = pos["legal"][i][:pos["n_legal"][i]]
        got = c.legal_policy(i)
        # same logits -> the device result equals the host formula bit for bit
        assert np.array_equal(got, oracle.softmax_policy(c.policy(i), ids))
        # and it is the reference's legal-move policy up to the fp32 noise of the logits
        assert np.abs(got - g["legal_probs"][i][:len(ids)]).max() <= 1e-6
        assert abs(got.sum() - 1.0) < 1e-5
    c.close()
    nw.close()


def test_temperature_compact_and_mixed_inputs():
    net, pos, n, g = load_case("cfg3_mini")
    nw = network.Network(net, "precision=fp16,max_batch=%d" % n)
    full = _run(nw, pos, 8, temperature=1.359)
    compact = _run(nw, pos, 8, temperature=1.359, compact=True)
    for i in range(8):
        ids = pos["legal"][i][:pos["n_legal"][i]]
        want = oracle.softmax_policy(full.policy(i), ids, 1.0 / 1.359)
        assert np.array_equal(full.legal_policy(i), want)
        assert np.array_equal(compact.legal_policy(i), want)
        assert abs(compact.get_q_val(i) - full.get_q_val(i)) == 0
    full.close()
    compact.close()
    # a position added without moves reports an empty move list; others are unaffected
    c = nw.new_computation()
    c.add_input(pos["masks"][0], pos["values"][0])
    c.add_input_with_moves(pos["masks"][1], pos["values"][1], pos["legal"][1][:pos["n_legal"][1]])
    c.compute_blocking()
    assert c.legal_policy(0).size == 0 and c.legal_policy(1).size == pos["n_legal"][1]
    with pytest.raises(_lib.B200Error):
        c.add_input_with_moves(pos["masks"][1], pos["values"][1], np.zeros(300, np.uint16))
    with pytest.raises(_lib.B200Error):
        c.add_input_with_moves(pos["masks"][1], pos["values"][1], np.array([1858], np.uint16))
    c.close()
    plain = nw.new_computation()
    plain.add_input(pos["masks"][0], pos["values"][0])
    plain.compute_blocking()
    with pytest.raises(_lib.B200Error):
        plain.legal_policy(0)
    plain.close()
    nw.close()
