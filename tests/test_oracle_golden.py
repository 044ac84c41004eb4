"""The numpy oracle against outputs recorded from the reference's own `blas` backend.

The goldens (tests/golden/golden_*.npz) were produced by oracle/_ref/ref_eval, i.e. the
reference's network_blas.cc compiled from its sources, on seeded networks and positions.
"""
import numpy as np
import pytest

from conftest import legal_logits, load_case, load_compact
from lc0_b200 import weights
from oracle import oracle

# fp32 summation-order noise between numpy and OpenBLAS; logits are O(1).
POLICY_ATOL = 2e-5
VALUE_ATOL = 5e-6


@pytest.mark.parametrize("name", ["cfg1_mini", "cfg2_mini", "cfg3_mini", "cfg4_mini", "cfg1", "cfg2", "cfg3",
                                  "cfg4_2layer", "cfg1_mini_tanh", "cfg3_mini_tanh", "cfg4_mini_outlier",
                                  "cfg3_mini_polenc"])
def test_oracle_matches_reference_blas(name):
    net, pos, n, g = load_case(name)
    meta, t = weights.flatten(net)
    out = oracle.forward(meta, t, pos["masks"][:n], pos["values"][:n])
    assert out["policy"].shape == (n, 1858)
    np.testing.assert_allclose(out["policy"], g["policy"], rtol=0, atol=POLICY_ATOL)
    np.testing.assert_allclose(out["q"], g["q"], rtol=0, atol=VALUE_ATOL)
    np.testing.assert_allclose(out["d"], g["d"], rtol=0, atol=VALUE_ATOL)
    np.testing.assert_allclose(out["m"], g["m"], rtol=0, atol=VALUE_ATOL)
    # the outputs must actually depend on the position
    assert np.abs(g["policy"] - g["policy"][0]).max() > 1e-4


def test_classical_value_goldens_use_the_tanh_branch():
    """VALUE_CLASSICAL networks: q = tanh(value), d = 0 (network_blas.cc:764-771)."""
    for name in ("cfg1_mini_tanh", "cfg3_mini_tanh"):
        net, pos, n, g = load_case(name)
        meta, t = weights.flatten(net)
        assert meta["value"] == 1  # VALUE_CLASSICAL
        assert np.all(g["d"] == 0) and np.all(np.abs(g["q"]) < 1) and np.abs(g["q"]).max() > 1e-3


def test_compact_large_batch_golden_matches_oracle_on_a_sample():
    """The 1024-position golden of the two-layer BT4-class net: the oracle on 24 positions spread over the set."""
    net, pos, n, g = load_compact("cfg4_2layer_b1024")
    assert n == 1024 and g["legal_logits"].shape == (1024, 256)
    meta, t = weights.flatten(net)
    idx = np.arange(0, 1024, 43)
    out = oracle.forward(meta, t, pos["masks"][idx], pos["values"][idx])
    sub = {k: pos[k][idx] for k in ("legal", "n_legal")}
    np.testing.assert_allclose(legal_logits(out["policy"], sub, len(idx)), g["legal_logits"][idx], rtol=0,
                               atol=POLICY_ATOL)
    np.testing.assert_allclose(out["q"], g["q"][idx], rtol=0, atol=VALUE_ATOL)
    np.testing.assert_allclose(out["m"], g["m"][idx], rtol=0, atol=VALUE_ATOL)


def test_oracle_empty_batch():
    net, pos, n, g = load_case("cfg3_mini")
    meta, t = weights.flatten(net)
    out = oracle.forward(meta, t, pos["masks"][:0], pos["values"][:0])
    assert out["policy"].shape == (0, 1858) and out["q"].shape == (0,)


def test_oracle_chunking_is_invisible():
    net, pos, n, g = load_case("cfg4_mini")
    meta, t = weights.flatten(net)
    a = oracle.forward(meta, t, pos["masks"][:7], pos["values"][:7], chunk=256)
    b = oracle.forward(meta, t, pos["masks"][:7], pos["values"][:7], chunk=3)
    np.testing.assert_allclose(a["policy"], b["policy"], atol=1e-6)


def test_mlh_option_zeroes_m():
    net, pos, n, g = load_case("cfg3_mini")
    meta, t = weights.flatten(net)
    out = oracle.forward(meta, t, pos["masks"][:4], pos["values"][:4], mlh=False)
    assert np.all(out["m"] == 0)


def test_expand_planes_bits():
    masks = np.zeros((1, 112), np.uint64)
    values = np.ones((1, 112), np.float32)
    masks[0, 0] = np.uint64(1)            # a1
    masks[0, 1] = np.uint64(1) << np.uint64(63)  # h8
    masks[0, 2] = np.uint64(0xFFFFFFFFFFFFFFFF)
    values[0, 2] = 0.25
    d = oracle.expand_planes(masks, values)
    assert d.shape == (1, 112, 64)
    assert d[0, 0, 0] == 1 and d[0, 0, 1:].sum() == 0
    assert d[0, 1, 63] == 1 and d[0, 1, :63].sum() == 0
    assert np.all(d[0, 2] == 0.25)
    assert d[0, 3:].sum() == 0


def test_activation_formulas():
    x = np.array([-3.0, -0.125, -0.1, 0.0, 0.5, 4.0], np.float32)
    sp = np.log1p(np.exp(x.astype(np.float64)))
    np.testing.assert_allclose(oracle.activate(x, oracle.ACT_MISH), x * np.tanh(sp), atol=1e-6)
    np.testing.assert_allclose(oracle.activate(x, oracle.ACT_RELU_2), np.where(x > 0, x * x, 0))
    np.testing.assert_allclose(oracle.activate(x, oracle.ACT_SWISH), x / (1 + np.exp(-x)), atol=1e-6)


@pytest.mark.parametrize("name", ["cfg1_mini", "cfg4_mini", "cfg3"])
def test_softmax_policy_restatement_is_bit_exact(name):
    """oracle.softmax_policy / fast_exp against the reference's own FastExp applied by ref_eval."""
    net, pos, n, g = load_case(name)
    for i in range(n):
        ids = pos["legal"][i][:pos["n_legal"][i]]
        got = oracle.softmax_policy(g["policy"][i], ids)
        assert np.array_equal(got, g["legal_probs"][i][:len(ids)])
        assert np.all(g["legal_probs"][i][len(ids):] == 0)


def test_fast_exp_edges():
    x = np.array([0.0, -1e-3, -0.5, -1.0, -10.0, -87.0, -88.0, -200.0], np.float32)
    y = oracle.fast_exp(x)
    assert y[0] == 1.0 and y[-1] == 0.0
    np.testing.assert_allclose(y[:6], np.exp(x[:6].astype(np.float64)), rtol=4e-3)  # FastExp is a 2nd-order fit
