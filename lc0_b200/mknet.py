"""Seeded synthetic lc0 networks for the benchmark configurations.

No lc0 weights file ships with the reference and none can be downloaded, so
every measured or tested network is random-initialised here and serialised as a
regular `net.proto` file (magic 0x1c0, per-layer FLOAT32 encoding) that the
reference's own loader accepts (neural/loader.cc:160-191).

Weight distributions: residual nets draw conv/FC weights from N(0, 1/fan_in) and
biases from N(0, 0.01^2); attention nets draw every matrix and bias from
N(0, 0.02^2), LayerNorm gammas and multiplicative gates from 1 + N(0, 0.02^2)
(the `*_mini` attention nets use 0.08 so that their narrow layers still produce
O(1) activations).
Values come from `numpy.random.Generator(PCG64(seed))` consumed in the field
order of the functions below, seed = 1000 + configuration number.

`*_mini` variants have the same structure at a fraction of the size; they exist
so that CPU-side and fp32 parity tests finish in seconds.
"""
import numpy as np

from . import netproto
from .netproto import NF, array_to_layer

CONFIGS = {
    # Residual CNN 10x128, SE ratio 4, classical policy, WDL, no moves-left (fp32, batch 64).
    "cfg1": dict(kind="resnet", seed=1001, blocks=10, filters=128, se=32, policy="classical",
                 policy_planes=32, value_planes=32, value_hidden=128, mlh=False,
                 input=NF.INPUT_CLASSICAL_112_PLANE),
    # Residual CNN 20x256, SE ratio 8, convolutional policy (80 planes), WDL + moves-left.
    "cfg2": dict(kind="resnet", seed=1002, blocks=20, filters=256, se=32, policy="conv",
                 policy_planes=80, value_planes=32, value_hidden=128, mlh=True, mlh_planes=8,
                 mlh_hidden=128, input=NF.INPUT_CLASSICAL_112_PLANE),
    # Small attention body: 10 layers, E=256, 8 heads, dff 512, PE_MAP, Mish, no smolgen.
    "cfg3": dict(kind="attn", seed=1003, layers=10, emb=256, heads=8, dff=512, multihead=False,
                 pe_dense=False, default_act=NF.DEFAULT_ACTIVATION_MISH, ffn_act=NF.ACTIVATION_MISH,
                 smolgen=None, pol_emb=256, pol_dmodel=256, value_planes=32, value_hidden=128,
                 mlh=True, mlh_planes=8, mlh_hidden=128, gating=True,
                 input=NF.INPUT_112_WITH_CASTLING_PLANE),
    # BT4-class: 15 layers, E=1024, 32 heads, dff 1536, ReLU^2, smolgen 32/256/256, PE_DENSE.
    "cfg4": dict(kind="attn", seed=1004, layers=15, emb=1024, heads=32, dff=1536, multihead=True,
                 pe_dense=True, dpe=512, emb_dff=1536, default_act=NF.DEFAULT_ACTIVATION_MISH,
                 ffn_act=NF.ACTIVATION_RELU_2, smolgen=dict(hc=32, hidden=256, gen=256,
                                                            act=NF.ACTIVATION_SWISH),
                 pol_emb=1024, pol_dmodel=1024, value_planes=32, value_hidden=128, mlh=True,
                 mlh_planes=8, mlh_hidden=128, gating=True, input=NF.INPUT_112_WITH_CASTLING_PLANE),
}
CONFIGS["cfg5"] = dict(CONFIGS["cfg4"])  # same net, different batch / position mix
CONFIGS["cfg1_mini"] = dict(CONFIGS["cfg1"], blocks=2, filters=32, se=8, policy_planes=8,
                            value_planes=8, value_hidden=32, seed=1011)
CONFIGS["cfg2_mini"] = dict(CONFIGS["cfg2"], blocks=2, filters=32, se=4, value_planes=8,
                            value_hidden=32, mlh_planes=4, mlh_hidden=16, seed=1012)
CONFIGS["cfg3_mini"] = dict(CONFIGS["cfg3"], layers=2, emb=64, heads=2, dff=96, pol_emb=64,
                            pol_dmodel=64, value_planes=8, value_hidden=32, mlh_planes=4,
                            mlh_hidden=16, std=0.08, seed=1013)
CONFIGS["cfg4_mini"] = dict(CONFIGS["cfg4"], layers=2, emb=128, heads=4, dff=192, dpe=32,
                            emb_dff=160, smolgen=dict(hc=8, hidden=32, gen=32,
                                                      act=NF.ACTIVATION_SWISH),
                            pol_emb=96, pol_dmodel=64, value_planes=8, value_hidden=32,
                            mlh_planes=4, mlh_hidden=16, std=0.08, seed=1014)
# BT4-class shapes (E=1024, 32 heads, dff 1536, smolgen 32/256/256) but only two layers: the
# tensor-core kernels see their production tile shapes while the CPU oracle still runs fast.
CONFIGS["cfg4_2layer"] = dict(CONFIGS["cfg4"], layers=2, seed=1024)
# Classical value head (one tanh output, VALUE_CLASSICAL / OUTPUT_CLASSICAL) on a residual and an attention body:
# the branch of the value head that WDL networks never take (network_blas.cc:764-771).
CONFIGS["cfg1_mini_tanh"] = dict(CONFIGS["cfg1_mini"], wdl=False, seed=1031)
CONFIGS["cfg3_mini_tanh"] = dict(CONFIGS["cfg3_mini"], wdl=False, mlh=False, seed=1033)
# Trained networks carry a few residual-stream channels that are orders of magnitude larger than the rest and rows
# whose mean is far from zero; random initialisation never produces either.  This variant plants both (LayerNorm
# gains / offsets of a few channels at 40..200, a common offset on the sub-layer biases), for the LayerNorm
# arithmetic of the 16-bit path.
CONFIGS["cfg4_mini_outlier"] = dict(CONFIGS["cfg4_mini"], outlier=True, seed=1044)
# Encoder layers inside the attention policy head (network_blas.cc:832-838), which no benchmark configuration has.
CONFIGS["cfg3_mini_polenc"] = dict(CONFIGS["cfg3_mini"], pol_layers=2, pol_heads=2, pol_dff=80, seed=1053)


class _Gen:
    def __init__(self, seed, encoding):
        self.rng = np.random.Generator(np.random.PCG64(seed))
        self.encoding = encoding

    def normal(self, n, std, mean=0.0):
        a = self.rng.standard_normal(int(n), dtype=np.float32) * np.float32(std) + np.float32(mean)
        return array_to_layer(a, self.encoding)


def _conv(g, cout, cin, k):
    fan_in = cin * k * k
    return {"weights": g.normal(cout * cin * k * k, fan_in ** -0.5), "biases": g.normal(cout, 0.01)}


def _fc(g, out, inp, std=None):
    std = inp ** -0.5 if std is None else std
    return g.normal(out * inp, std)


def _make_resnet(c, g):
    C = c["filters"]
    w = {"input": _conv(g, C, 112, 3), "residual": []}
    for _ in range(c["blocks"]):
        res = {"conv1": _conv(g, C, C, 3), "conv2": _conv(g, C, C, 3)}
        if c["se"]:
            k = c["se"]
            res["se"] = {"w1": _fc(g, k, C), "b1": g.normal(k, 0.01),
                         "w2": _fc(g, 2 * C, k), "b2": g.normal(2 * C, 0.01)}
        w["residual"].append(res)
    if c["policy"] == "classical":
        P = c["policy_planes"]
        w["policy"] = _conv(g, P, C, 1)
        w["ip_pol_w"] = _fc(g, 1858, P * 64)
        w["ip_pol_b"] = g.normal(1858, 0.01)
    else:
        w["policy1"] = _conv(g, C, C, 3)
        w["policy"] = _conv(g, c["policy_planes"], C, 3)
    V, VH = c["value_planes"], c["value_hidden"]
    w["value"] = _conv(g, V, C, 1)
    w["ip1_val_w"] = _fc(g, VH, V * 64)
    w["ip1_val_b"] = g.normal(VH, 0.01)
    outs = 3 if c.get("wdl", True) else 1
    w["ip2_val_w"] = _fc(g, outs, VH)
    w["ip2_val_b"] = g.normal(outs, 0.01)
    if c["mlh"]:
        M, MH = c["mlh_planes"], c["mlh_hidden"]
        w["moves_left"] = _conv(g, M, C, 1)
        w["ip1_mov_w"] = _fc(g, MH, M * 64)
        w["ip1_mov_b"] = g.normal(MH, 0.01)
        w["ip2_mov_w"] = _fc(g, 1, MH)
        w["ip2_mov_b"] = g.normal(1, 0.01, 1.0)
    nf = {"input": c["input"], "output": NF.OUTPUT_WDL if c.get("wdl", True) else NF.OUTPUT_CLASSICAL,
          "network": NF.NETWORK_SE_WITH_HEADFORMAT,
          "policy": NF.POLICY_CLASSICAL if c["policy"] == "classical" else NF.POLICY_CONVOLUTION,
          "value": NF.VALUE_WDL if c.get("wdl", True) else NF.VALUE_CLASSICAL,
          "moves_left": NF.MOVES_LEFT_V1 if c["mlh"] else NF.MOVES_LEFT_NONE,
          "default_activation": NF.DEFAULT_ACTIVATION_RELU}
    return w, nf


def _make_attn(c, g):
    S = c.get("std", 0.02)
    E, H, F, L = c["emb"], c["heads"], c["dff"], c["layers"]
    w = {}
    if c["pe_dense"]:
        dpe = c["dpe"]
        w["ip_emb_preproc_w"] = g.normal(64 * dpe * 64 * 12, S)
        w["ip_emb_preproc_b"] = g.normal(64 * dpe, S)
        in_ch = 112 + dpe
    else:
        in_ch = 112 + 64
    w["ip_emb_w"] = g.normal(E * in_ch, S)
    w["ip_emb_b"] = g.normal(E, S)
    if c["pe_dense"]:
        w["ip_emb_ln_gammas"] = g.normal(E, S, 1.0)
        w["ip_emb_ln_betas"] = g.normal(E, S)
    if c["gating"]:
        w["ip_mult_gate"] = g.normal(E * 64, S, 1.0)
        w["ip_add_gate"] = g.normal(E * 64, S)
    if c["pe_dense"]:
        EF = c["emb_dff"]
        w["ip_emb_ffn"] = {"dense1_w": g.normal(EF * E, S), "dense1_b": g.normal(EF, S),
                           "dense2_w": g.normal(E * EF, S), "dense2_b": g.normal(E, S)}
        w["ip_emb_ffn_ln_gammas"] = g.normal(E, S, 1.0)
        w["ip_emb_ffn_ln_betas"] = g.normal(E, S)
    sg = c["smolgen"]
    w["encoder"] = []
    for _ in range(L):
        mha = {"q_w": g.normal(E * E, S), "q_b": g.normal(E, S), "k_w": g.normal(E * E, S),
               "k_b": g.normal(E, S), "v_w": g.normal(E * E, S), "v_b": g.normal(E, S),
               "dense_w": g.normal(E * E, S), "dense_b": g.normal(E, S)}
        if sg:
            hc, hid, gen = sg["hc"], sg["hidden"], sg["gen"]
            mha["smolgen"] = {
                "compress": g.normal(hc * E, S),
                "dense1_w": g.normal(hid * 64 * hc, S), "dense1_b": g.normal(hid, S),
                "ln1_gammas": g.normal(hid, S, 1.0), "ln1_betas": g.normal(hid, S),
                "dense2_w": g.normal(H * gen * hid, S), "dense2_b": g.normal(H * gen, S),
                "ln2_gammas": g.normal(H * gen, S, 1.0), "ln2_betas": g.normal(H * gen, S)}
        w["encoder"].append({
            "mha": mha, "ln1_gammas": g.normal(E, S, 1.0), "ln1_betas": g.normal(E, S),
            "ffn": {"dense1_w": g.normal(F * E, S), "dense1_b": g.normal(F, S),
                    "dense2_w": g.normal(E * F, S), "dense2_b": g.normal(E, S)},
            "ln2_gammas": g.normal(E, S, 1.0), "ln2_betas": g.normal(E, S)})
    w["headcount"] = H
    if sg:
        w["smolgen_w"] = g.normal(4096 * sg["gen"], S)
    PE, PD = c["pol_emb"], c["pol_dmodel"]
    pol = {"ip2_pol_w": g.normal(PD * PE, S), "ip2_pol_b": g.normal(PD, S),
           "ip3_pol_w": g.normal(PD * PE, S), "ip3_pol_b": g.normal(PD, S),
           "ip4_pol_w": g.normal(4 * PD, S)}
    if c.get("pol_layers"):
        PF = c["pol_dff"]
        pol["pol_headcount"] = c["pol_heads"]
        pol["pol_encoder"] = [{
            "mha": {"q_w": g.normal(PE * PE, S), "q_b": g.normal(PE, S), "k_w": g.normal(PE * PE, S),
                    "k_b": g.normal(PE, S), "v_w": g.normal(PE * PE, S), "v_b": g.normal(PE, S),
                    "dense_w": g.normal(PE * PE, S), "dense_b": g.normal(PE, S)},
            "ln1_gammas": g.normal(PE, S, 1.0), "ln1_betas": g.normal(PE, S),
            "ffn": {"dense1_w": g.normal(PF * PE, S), "dense1_b": g.normal(PF, S),
                    "dense2_w": g.normal(PE * PF, S), "dense2_b": g.normal(PE, S)},
            "ln2_gammas": g.normal(PE, S, 1.0), "ln2_betas": g.normal(PE, S)} for _ in range(c["pol_layers"])]
    V, VH = c["value_planes"], c["value_hidden"]
    val = {"ip_val_w": g.normal(V * E, S), "ip_val_b": g.normal(V, S),
           "ip1_val_w": g.normal(VH * V * 64, S), "ip1_val_b": g.normal(VH, S),
           "ip2_val_w": g.normal((3 if c.get("wdl", True) else 1) * VH, S),
           "ip2_val_b": g.normal(3 if c.get("wdl", True) else 1, S)}
    if c["multihead"]:
        w["policy_heads"] = {"ip_pol_w": g.normal(PE * E, S), "ip_pol_b": g.normal(PE, S),
                             "vanilla": pol}
        w["value_heads"] = {"winner": val}
    else:
        w["ip_pol_w"] = g.normal(PE * E, S)
        w["ip_pol_b"] = g.normal(PE, S)
        w.update(pol)
        w.update(val)
    if c["mlh"]:
        M, MH = c["mlh_planes"], c["mlh_hidden"]
        w["ip_mov_w"] = g.normal(M * E, S)
        w["ip_mov_b"] = g.normal(M, S)
        w["ip1_mov_w"] = g.normal(MH * M * 64, S)
        w["ip1_mov_b"] = g.normal(MH, S)
        w["ip2_mov_w"] = g.normal(MH, S)
        w["ip2_mov_b"] = g.normal(1, S, 0.5)
    nf = {"input": c["input"], "output": NF.OUTPUT_WDL if c.get("wdl", True) else NF.OUTPUT_CLASSICAL,
          "network": NF.NETWORK_ATTENTIONBODY_WITH_MULTIHEADFORMAT if c["multihead"]
          else NF.NETWORK_ATTENTIONBODY_WITH_HEADFORMAT,
          "policy": NF.POLICY_ATTENTION, "value": NF.VALUE_WDL if c.get("wdl", True) else NF.VALUE_CLASSICAL,
          "moves_left": NF.MOVES_LEFT_V1 if c["mlh"] else NF.MOVES_LEFT_NONE,
          "default_activation": c["default_act"], "ffn_activation": c["ffn_act"],
          "input_embedding": NF.INPUT_EMBEDDING_PE_DENSE if c["pe_dense"]
          else NF.INPUT_EMBEDDING_PE_MAP}
    if sg:
        nf["smolgen_activation"] = sg["act"]
    if c.get("outlier"):
        _plant_outliers(w, g.encoding)
    return w, nf


def _plant_outliers(w, encoding):
    """Large LayerNorm gains / offsets on a few channels and a common offset on the sub-layer output biases of every
    encoder layer (see CONFIGS["cfg4_mini_outlier"])."""
    def edit(holder, key, fn):
        a = netproto.layer_to_array(holder[key]).copy()
        fn(a)
        holder[key] = array_to_layer(a, encoding)

    for i, enc in enumerate(w["encoder"]):
        def bump(a, ch, v):
            a[ch % a.size] = v
        edit(enc, "ln1_gammas", lambda a: bump(a, 3 + 7 * i, 12.0))
        edit(enc, "ln1_betas", lambda a: bump(a, 3 + 7 * i, 20.0))
        edit(enc, "ln2_gammas", lambda a: bump(a, 11 + 5 * i, 16.0))
        edit(enc, "ln2_betas", lambda a: bump(a, 11 + 5 * i, -24.0))
        edit(enc["mha"], "dense_b", lambda a: a.__iadd__(np.float32(5.0)))
        edit(enc["ffn"], "dense2_b", lambda a: a.__isub__(np.float32(7.0)))


def make_net(name, encoding=netproto.FLOAT32, **overrides):
    """Build the `Net` dict of configuration `name` (a key of CONFIGS)."""
    c = dict(CONFIGS[name], **overrides)
    g = _Gen(c["seed"], encoding)
    w, nf = (_make_resnet if c["kind"] == "resnet" else _make_attn)(c, g)
    return {"magic": netproto.WEIGHT_MAGIC, "license": "synthetic random-init network",
            "min_version": {"major": 0, "minor": 30, "patch": 0},
            "format": {"weights_encoding": 1, "network_format": nf}, "weights": w}


def write_net(name, path, **kw):
    net = make_net(name, **kw)
    netproto.write_net(path, net, compress=path.endswith(".gz"))
    return net


if __name__ == "__main__":
    import sys
    write_net(sys.argv[1], sys.argv[2])
