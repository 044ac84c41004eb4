"""Weight-file codec, loader checks and the MultiHeadWeights-style flattening (host logic, CPU only)."""
import gzip
import os

import numpy as np
import pytest

from lc0_b200 import mknet, netproto, weights
from lc0_b200.netproto import NF


def test_roundtrip_and_gzip(tmp_path):
    net = mknet.make_net("cfg4_mini")
    p = str(tmp_path / "n.pb.gz")
    netproto.write_net(p, net)
    assert open(p, "rb").read(2) == b"\x1f\x8b"
    back = netproto.load_net(p)
    m1, t1 = weights.flatten(netproto.parse_net(netproto.encode("Net", net)))
    m2, t2 = weights.flatten(back)
    assert m1 == m2 and t1.keys() == t2.keys()
    for k in t1:
        assert np.array_equal(t1[k], t2[k])
    p2 = str(tmp_path / "n.pb")
    netproto.write_net(p2, net, compress=False)
    assert netproto.load_net(p2)["magic"] == 0x1C0


@pytest.mark.parametrize("enc,tol", [(netproto.FLOAT32, 0.0), (netproto.FLOAT16, 1e-3),
                                     (netproto.BFLOAT16, 1e-2), (netproto.LINEAR16, 1e-4)])
def test_layer_encodings(enc, tol):
    a = np.random.default_rng(0).standard_normal(1000).astype(np.float32)
    layer = netproto.array_to_layer(a, enc)
    b = netproto.layer_to_array(netproto.decode("Layer", netproto.encode("Layer", layer)))
    assert b.dtype == np.float32 and np.abs(a - b).max() <= tol * max(1.0, np.abs(a).max())


def test_layer_without_encoding_is_linear16():
    layer = {"min_val": -1.0, "max_val": 3.0, "params": np.array([0, 65535, 32768], "<u2").tobytes()}
    np.testing.assert_allclose(netproto.layer_to_array(layer), [-1.0, 3.0, 1.0], atol=1e-4)


def test_loader_rejections():
    good = netproto.encode("Net", mknet.make_net("cfg1_mini"))
    with pytest.raises(ValueError, match="too small"):
        netproto.parse_net(b"x")
    net = mknet.make_net("cfg1_mini")
    net["magic"] = 0x1C1
    with pytest.raises(ValueError, match="bad header"):
        netproto.parse_net(netproto.encode("Net", net))
    net = mknet.make_net("cfg1_mini")
    net["min_version"] = {"major": 0, "minor": 99, "patch": 0}
    with pytest.raises(ValueError, match="lc0 version"):
        netproto.parse_net(netproto.encode("Net", net))
    net = mknet.make_net("cfg1_mini")
    net["format"]["weights_encoding"] = 0
    with pytest.raises(ValueError, match="unsupported encoding"):
        netproto.parse_net(netproto.encode("Net", net))
    with pytest.raises(ValueError):
        netproto.parse_net(good[:len(good) // 2])  # truncated


def test_format_fixups():
    net = netproto.parse_net(netproto.encode("Net", mknet.make_net("cfg3_mini")))
    nf = net["format"]["network_format"]
    assert nf["network"] == NF.NETWORK_ATTENTIONBODY_WITH_HEADFORMAT
    assert nf["input_embedding"] == NF.INPUT_EMBEDDING_PE_MAP
    old = mknet.make_net("cfg1_mini")
    old["format"]["network_format"]["network"] = NF.NETWORK_SE
    fixed = netproto.parse_net(netproto.encode("Net", old))["format"]["network_format"]
    assert fixed["network"] == NF.NETWORK_SE_WITH_HEADFORMAT and fixed["policy"] == NF.POLICY_CLASSICAL


def test_batchnorm_folding():
    rng = np.random.default_rng(1)
    cout, cin = 4, 3
    w = rng.standard_normal(cout * cin * 9).astype(np.float32)
    means, std = rng.standard_normal(cout).astype(np.float32), rng.random(cout).astype(np.float32) + 0.5
    gam, bet = rng.standard_normal(cout).astype(np.float32), rng.standard_normal(cout).astype(np.float32)
    L = netproto.array_to_layer
    blk = {"weights": L(w), "bn_means": L(means), "bn_stddivs": L(std), "bn_gammas": L(gam), "bn_betas": L(bet)}
    fw, fb = weights._conv_block(blk)
    x = rng.standard_normal(cin * 9).astype(np.float32)
    raw = w.reshape(cout, -1) @ x
    want = gam * (raw - means) / np.sqrt(std + 1e-5) + bet
    np.testing.assert_allclose(fw.reshape(cout, -1) @ x + fb, want, rtol=1e-5, atol=1e-5)


def test_head_selection_errors():
    net = netproto.parse_net(netproto.encode("Net", mknet.make_net("cfg4_mini")))
    with pytest.raises(weights.WeightsError, match="policy head"):
        weights.flatten(net, policy_head="soft")
    with pytest.raises(weights.WeightsError, match="value head"):
        weights.flatten(net, value_head="q")
    net["weights"]["encoder"][0]["mha"]["rpe_q"] = netproto.array_to_layer(np.zeros(4))
    with pytest.raises(weights.WeightsError, match="RPE"):
        weights.flatten(net)


def test_activation_resolution():
    meta, _ = weights.flatten(netproto.parse_net(netproto.encode("Net", mknet.make_net("cfg4_mini"))))
    assert meta["default_activation"] == NF.ACTIVATION_MISH
    assert meta["ffn_activation"] == NF.ACTIVATION_RELU_2 and meta["smolgen_activation"] == NF.ACTIVATION_SWISH
    meta, _ = weights.flatten(netproto.parse_net(netproto.encode("Net", mknet.make_net("cfg1_mini"))))
    assert meta["default_activation"] == NF.ACTIVATION_RELU and meta["ffn_activation"] == NF.ACTIVATION_RELU


def test_seeded_nets_are_deterministic():
    a = netproto.encode("Net", mknet.make_net("cfg3_mini"))
    b = netproto.encode("Net", mknet.make_net("cfg3_mini"))
    assert a == b
