"""Flatten a parsed lc0 `Net` into the named fp32 tensors the backend consumes.

Restates what the reference does between the weights file and a backend:
`MultiHeadWeights` construction (neural/network_legacy.cc:33-307: per-layer
decoding, batch-norm folding into convolution weights and biases, selection of
legacy single-head fields versus the multi-head containers) and the activation
/ format resolution each backend performs (backends/blas/network_blas.cc:996-1028,
:1051-1063).  The result is `(meta, tensors)`:

* `meta`: dict of ints (format enums resolved to concrete activation functions,
  head counts), passed to the C-ABI with `b200_builder_set_int`;
* `tensors`: dict name -> float32 ndarray, passed with `b200_builder_add_tensor`.
  All dense weights keep the file's `[out][in]` row-major layout, convolution
  weights `[Cout][Cin][3][3]`.
"""
import numpy as np

from .netproto import NF, layer_to_array

_BN_EPS = np.float32(1e-5)  # neural/network_legacy.cc:30


class WeightsError(ValueError):
    pass


def _vec(msg, name):
    return layer_to_array(msg.get(name)) if msg else np.zeros(0, np.float32)


def _conv_block(block):
    """ConvBlock with batch norm folded (neural/network_legacy.cc:78-133)."""
    if not block:
        return None
    w = _vec(block, "weights").copy()
    b = _vec(block, "biases").copy()
    if w.size == 0:
        return None
    gam, bet = _vec(block, "bn_gammas").copy(), _vec(block, "bn_betas").copy()
    mean, std = _vec(block, "bn_means").copy(), _vec(block, "bn_stddivs")
    if bet.size == 0:
        bet = np.zeros(mean.size, np.float32)
        gam = np.ones(mean.size, np.float32)
    if b.size == 0:
        b = np.zeros(mean.size, np.float32)
    if mean.size:
        gam = gam * (np.float32(1.0) / np.sqrt(std + _BN_EPS))
        mean = mean - b
        outputs = b.size
        w = (w.reshape(outputs, -1) * gam[:, None]).reshape(-1)
        b = -gam * mean + bet
    return w.astype(np.float32), b.astype(np.float32)


def _put(t, name, arr):
    if arr is not None and arr.size:
        t[name] = np.ascontiguousarray(arr, np.float32)


def _put_conv(t, prefix, block):
    cb = _conv_block(block)
    if cb is not None:
        t[prefix + ".weights"], t[prefix + ".biases"] = cb


def _put_encoder(t, prefix, enc):
    mha = enc.get("mha", {})
    if any(k in mha for k in ("rpe_q", "rpe_k", "rpe_v")):
        raise WeightsError("RPE weights file not supported.")  # network_legacy.cc:146-148
    for k in ("q_w", "q_b", "k_w", "k_b", "v_w", "v_b", "dense_w", "dense_b"):
        _put(t, "%s.mha.%s" % (prefix, k), _vec(mha, k))
    if "smolgen" in mha:
        sg = mha["smolgen"]
        for k in ("compress", "dense1_w", "dense1_b", "ln1_gammas", "ln1_betas", "dense2_w",
                  "dense2_b", "ln2_gammas", "ln2_betas"):
            _put(t, "%s.mha.smolgen.%s" % (prefix, k), _vec(sg, k))
    for k in ("ln1_gammas", "ln1_betas", "ln2_gammas", "ln2_betas"):
        _put(t, "%s.%s" % (prefix, k), _vec(enc, k))
    ffn = enc.get("ffn", {})
    for k in ("dense1_w", "dense1_b", "dense2_w", "dense2_b"):
        _put(t, "%s.ffn.%s" % (prefix, k), _vec(ffn, k))


def resolve_activations(nf):
    """(default, smolgen, ffn) activation functions (network_blas.cc:1010-1028)."""
    default = NF.ACTIVATION_MISH if nf.get("default_activation", 0) == NF.DEFAULT_ACTIVATION_MISH \
        else NF.ACTIVATION_RELU
    smol = nf.get("smolgen_activation", 0) or default
    ffn = nf.get("ffn_activation", 0) or default
    return default, smol, ffn


def flatten(net, policy_head="vanilla", value_head="winner"):
    """Return (meta, tensors) for a parsed `Net` (see module docstring)."""
    if "weights" not in net:
        raise WeightsError("The b200 backend requires a network file with weights.")
    w = net["weights"]
    nf = net.get("format", {}).get("network_format", {})
    network = nf.get("network", 0)
    if network not in (NF.NETWORK_CLASSICAL_WITH_HEADFORMAT, NF.NETWORK_SE_WITH_HEADFORMAT,
                       NF.NETWORK_ATTENTIONBODY_WITH_HEADFORMAT,
                       NF.NETWORK_ATTENTIONBODY_WITH_MULTIHEADFORMAT):
        raise WeightsError("Network format %d is not supported by the b200 backend." % network)
    if nf.get("policy", 0) not in (NF.POLICY_CLASSICAL, NF.POLICY_CONVOLUTION, NF.POLICY_ATTENTION):
        raise WeightsError("Policy format %d is not supported by the b200 backend." % nf.get("policy", 0))
    if nf.get("value", 0) not in (NF.VALUE_CLASSICAL, NF.VALUE_WDL):
        raise WeightsError("Value format %d is not supported by the b200 backend." % nf.get("value", 0))
    if nf.get("moves_left", 0) not in (NF.MOVES_LEFT_NONE, NF.MOVES_LEFT_V1):
        raise WeightsError("Moves left head format %d is not supported." % nf.get("moves_left", 0))
    if nf.get("input_embedding", 0) not in (0, 1, 2):
        raise WeightsError("Input embedding %d is not supported." % nf.get("input_embedding", 0))

    t = {}
    _put_conv(t, "input", w.get("input"))
    for i, res in enumerate(w.get("residual", [])):
        _put_conv(t, "residual.%d.conv1" % i, res.get("conv1"))
        _put_conv(t, "residual.%d.conv2" % i, res.get("conv2"))
        if "se" in res:
            for k in ("w1", "b1", "w2", "b2"):
                _put(t, "residual.%d.se.%s" % (i, k), _vec(res["se"], k))
    for k in ("ip_emb_preproc_w", "ip_emb_preproc_b", "ip_emb_w", "ip_emb_b", "ip_emb_ln_gammas",
              "ip_emb_ln_betas", "ip_mult_gate", "ip_add_gate", "ip_emb_ffn_ln_gammas",
              "ip_emb_ffn_ln_betas", "ip_mov_w", "ip_mov_b", "ip1_mov_w", "ip1_mov_b", "ip2_mov_w",
              "ip2_mov_b", "smolgen_w"):
        _put(t, k, _vec(w, k))
    ffn = w.get("ip_emb_ffn", {})
    for k in ("dense1_w", "dense1_b", "dense2_w", "dense2_b"):
        _put(t, "ip_emb_ffn." + k, _vec(ffn, k))
    for i, enc in enumerate(w.get("encoder", [])):
        _put_encoder(t, "encoder.%d" % i, enc)
    _put_conv(t, "moves_left", w.get("moves_left"))

    # ---- policy head selection (network_legacy.cc:232-284) ----
    pol_headcount = 0
    if "policy_heads" in w:
        ph = w["policy_heads"]
        key = {"vanilla": "vanilla", "optimistic": "optimistic_st", "soft": "soft",
               "opponent": "opponent"}.get(policy_head)
        if key is None or (key != "vanilla" and key not in ph):
            raise WeightsError("The policy head you specified '%s' does not exist in this net." % policy_head)
        head = ph.get(key, {})
        shared_w = _vec(ph, "ip_pol_w") if "ip_pol_w" in ph else _vec(w, "ip_pol_w")
        shared_b = _vec(ph, "ip_pol_b") if "ip_pol_b" in ph else _vec(w, "ip_pol_b")
        own_w, own_b = _vec(head, "ip_pol_w"), _vec(head, "ip_pol_b")
        _put(t, "policy.ip_pol_w", own_w if own_w.size else shared_w)
        _put(t, "policy.ip_pol_b", own_b if own_b.size else shared_b)
        src = head
    else:
        if policy_head != "vanilla":
            raise WeightsError("The policy head you specified '%s' does not exist in this net." % policy_head)
        if not any(k in w for k in ("policy", "policy1", "ip_pol_w")):
            raise WeightsError("Could not find valid policy head weights.")
        _put(t, "policy.ip_pol_w", _vec(w, "ip_pol_w"))
        _put(t, "policy.ip_pol_b", _vec(w, "ip_pol_b"))
        src = w
    for k in ("ip2_pol_w", "ip2_pol_b", "ip3_pol_w", "ip3_pol_b", "ip4_pol_w"):
        _put(t, "policy." + k, _vec(src, k))
    _put_conv(t, "policy.policy1", src.get("policy1"))
    _put_conv(t, "policy.policy", src.get("policy"))
    pol_headcount = src.get("pol_headcount", 0)
    for i, enc in enumerate(src.get("pol_encoder", [])):
        _put_encoder(t, "policy.pol_encoder.%d" % i, enc)

    # ---- value head selection (network_legacy.cc:286-306) ----
    if "value_heads" in w:
        vh = w["value_heads"]
        if value_head not in ("winner", "q", "st") or (value_head != "winner" and value_head not in vh):
            raise WeightsError("The value head you specified '%s' does not exist in this net." % value_head)
        vsrc = vh.get(value_head, {})
    else:
        if value_head != "winner":
            raise WeightsError("The value head you specified '%s' does not exist in this net." % value_head)
        if not any(k in w for k in ("value", "ip_val_w")):
            raise WeightsError("Could not find valid value head weights.")
        vsrc = w
    for k in ("ip_val_w", "ip_val_b", "ip1_val_w", "ip1_val_b", "ip2_val_w", "ip2_val_b"):
        _put(t, "value." + k, _vec(vsrc, k))
    _put_conv(t, "value.value", vsrc.get("value"))

    default, smol, ffn_act = resolve_activations(nf)
    meta = {
        "input_format": nf.get("input", 0),
        "output_format": nf.get("output", 0),
        "network": network,
        "policy": nf.get("policy", 0),
        "value": nf.get("value", 0),
        "moves_left": nf.get("moves_left", 0),
        "default_activation": default,
        "smolgen_activation": smol,
        "ffn_activation": ffn_act,
        "input_embedding": nf.get("input_embedding", 0),
        "headcount": w.get("headcount", 0),
        "pol_headcount": pol_headcount,
    }
    return meta, t
