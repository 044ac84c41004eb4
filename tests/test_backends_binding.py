"""The `lczero.backends`-shaped module (lc0_b200/backends.py) against the interface of src/python/weights.h."""
import os

import numpy as np
import pytest

from conftest import load_case
from lc0_b200 import backends, mknet
from oracle import oracle


@pytest.fixture(scope="module")
def weights_file(tmp_path_factory):
    path = str(tmp_path_factory.mktemp("nets") / "cfg4_mini.pb.gz")
    mknet.write_net("cfg4_mini", path)
    return path


def test_weights_accessors(weights_file, tmp_path):
    w = backends.Weights(weights_file)
    assert w.filename() == weights_file and w.license().startswith("synthetic")
    assert w.min_version() == "0.30.0"
    assert (w.input_format(), w.policy_format(), w.value_format(), w.moves_left_format()) == (2, 3, 2, 1)
    assert w.blocks() == 0
    with pytest.raises(backends.LczeroException, match="does not use residual blocks"):
        w.filters()
    res = str(tmp_path / "cfg1_mini.pb.gz")
    mknet.write_net("cfg1_mini", res)
    wr = backends.Weights(res)
    assert wr.blocks() == 2 and wr.filters() == 32
    with pytest.raises(backends.LczeroException):
        backends.Weights(str(tmp_path / "missing.pb.gz"))
    with pytest.raises(backends.LczeroException):
        backends.Weights(None)


def test_input_planes():
    i = backends.Input()
    assert i.mask(0) == 0 and i.val(111) == 0.0
    i.set_mask(3, 0xFFFF00000000FFFF)
    i.set_val(3, 0.5)
    j = i.clone()
    i.set_mask(3, 1)
    assert j.mask(3) == 0xFFFF00000000FFFF and j.val(3) == 0.5 and i.mask(3) == 1
    for bad in (-1, 112):
        with pytest.raises(backends.LczeroException, match="Plane index"):
            i.set_mask(bad, 0)
        with pytest.raises(backends.LczeroException, match="Plane index"):
            i.val(bad)


def test_output_softmax_is_the_reference_arithmetic():
    """p_softmax equals the legal-move softmax the reference's own FastExp produced (recorded by ref_eval), bit for
    bit, and the module's FastExp equals the oracle's restatement."""
    net, pos, n, g = load_case("cfg4_mini")
    for s in range(n):
        ids = [int(k) for k in pos["legal"][s][:pos["n_legal"][s]]]
        o = backends.Output(g["policy"][s], g["q"][s], g["d"][s], g["m"][s])
        assert np.array_equal(np.array(o.p_softmax(*ids), np.float32), g["legal_probs"][s][:len(ids)])
        assert o.p_raw(*ids[:3]) == tuple(float(g["policy"][s][k]) for k in ids[:3])
    assert o.p_softmax() == ()
    with pytest.raises(backends.LczeroException, match="between 0 and 1857"):
        o.p_raw(1858)
    x = np.linspace(-90, 0, 1001).astype(np.float32)
    assert np.array_equal(backends._fast_exp(x), oracle.fast_exp(x))


def test_backend_names_and_errors(weights_file):
    assert "b200" in backends.Backend.available_backends()
    w = backends.Weights(weights_file)
    with pytest.raises(backends.LczeroException, match="Unknown backend"):
        backends.Backend(weights=w, backend="cudnn")
    with pytest.raises(backends.LczeroException, match="requires a network file"):
        backends.Backend()
    with pytest.raises(backends.LczeroException, match="Unknown backend option"):
        backends.Backend(weights=w, options="no_such_option=1")


@pytest.mark.gpu
def test_backend_evaluate_matches_reference(weights_file):
    """The recorded reference outputs of the mini BT4-class network through Weights / Input / Backend.evaluate / Output."""
    net, pos, n, g = load_case("cfg4_mini")
    w = backends.Weights(weights_file)
    b = backends.Backend(weights=w, backend="b200-fp32", options="max_batch=%d" % n)
    assert b.capabilities().input_format() == 2 and b.capabilities().moves_left_format() == 1
    inputs = []
    for s in range(n):
        i = backends.Input()
        for p in range(112):
            i.set_mask(p, int(pos["masks"][s][p]))
            i.set_val(p, float(pos["values"][s][p]))
        inputs.append(i)
    outs = b.evaluate(*inputs)
    assert len(outs) == n and b.evaluate() == ()
    for s, o in enumerate(outs):
        ids = [int(k) for k in pos["legal"][s][:pos["n_legal"][s]]]
        assert abs(o.q() - g["q"][s]) < 1e-5 and abs(o.d() - g["d"][s]) < 1e-5 and abs(o.m() - g["m"][s]) < 1e-5
        np.testing.assert_allclose(o.p_raw(*ids), g["policy"][s][ids], atol=2e-5)
        np.testing.assert_allclose(o.p_softmax(*ids), g["legal_probs"][s][:len(ids)], atol=1e-5)
    half = backends.Backend(weights=w, backend="b200", options="max_batch=4")
    o16 = half.evaluate(*inputs[:3])
    assert len(o16) == 3 and abs(o16[1].q() - g["q"][1]) < 2e-3
    with pytest.raises(backends.LczeroException, match="max_batch"):
        half.evaluate(*inputs[:5])
