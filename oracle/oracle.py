"""CPU oracle: numpy fp32 restatement of lc0's `blas` backend forward pass.

TEST INFRASTRUCTURE ONLY.  Nothing under `lc0_b200/` may import this module; it
is used by `tests/`, by `__graft_entry__.smoke()` and by the `cpu_baseline` leg
of `bench.py` as the checker for the CUDA path, never as a fallback.

Pinning: this restatement is checked against outputs of the reference's own
`blas` backend (the binary `oracle/_ref/ref_eval`, compiled from the reference
sources by `oracle/build_ref.py`) on seeded networks and seeded positions; the
recorded outputs live in `tests/golden/*.npz` (made by `tests/golden/make_golden.py`).
The reference itself has no numeric test vectors for this path.

Every function cites the reference code it follows (paths relative to the lc0
source tree).  Inputs are the flattened tensors of `lc0_b200.weights.flatten`.
"""
import numpy as np

F32 = np.float32
# ActivationFunction values (neural/tables/activation_function.h:24-35).
ACT_MISH, ACT_RELU, ACT_NONE, ACT_TANH, ACT_SIGMOID, ACT_SELU, ACT_SWISH, ACT_RELU_2 = 1, 2, 3, 4, 5, 6, 7, 8


# --- tables (generated independently of the product's C++ generator) ----------------
def _tables():
    from oracle import tables  # pure-python chess geometry
    return tables


def expand_planes(masks, values):
    """`BlasComputation::EncodePlanes` (backends/blas/network_blas.cc:973-981):
    dense[n][p][sq] = values[n][p] if bit sq of masks[n][p] else 0."""
    masks = np.asarray(masks, np.uint64).reshape(-1, 112)
    values = np.asarray(values, F32).reshape(-1, 112)
    bits = (masks[:, :, None] >> np.arange(64, dtype=np.uint64)[None, None, :]) & np.uint64(1)
    return np.where(bits != 0, values[:, :, None], F32(0)).astype(F32)


def activate(x, act):
    """`Activate` (backends/shared/activation.cc:51-94)."""
    x = np.asarray(x, F32)
    if act == ACT_NONE:
        return x
    if act == ACT_RELU:
        return np.maximum(x, F32(0))
    if act == ACT_RELU_2:
        return np.where(x > 0, x * x, F32(0)).astype(F32)
    if act == ACT_MISH:
        # mish(x) = x*n/(n+2), n = e^2x + 2e^x, with the reference's stable branch.
        with np.errstate(over="ignore", invalid="ignore"):
            e = np.exp(x)
            n = e * e + F32(2) * e
            d = x / (n + F32(2))
            return np.where(x <= F32(-0.125), n * d, x - F32(2) * d).astype(F32)
    if act == ACT_TANH:
        return np.tanh(x)
    if act == ACT_SIGMOID:
        return (F32(1) / (F32(1) + np.exp(-x))).astype(F32)
    if act == ACT_SELU:
        alpha, scale = F32(1.67326324), F32(1.05070098)
        with np.errstate(over="ignore"):
            return np.where(x > 0, scale * x, scale * alpha * (np.exp(x) - F32(1))).astype(F32)
    if act == ACT_SWISH:
        return (x / (F32(1) + np.exp(-x))).astype(F32)
    raise ValueError("unsupported activation function %r" % (act,))


def fc(x, w, b, act, outputs):
    """`FullyConnectedLayer::Forward1D` (backends/blas/fully_connected_layer.cc:50-106):
    y = act(x . W^T + b) with W stored [out][in]."""
    x = np.asarray(x, F32)
    inputs = x.shape[-1]
    y = x @ w.reshape(outputs, inputs).T
    if b is not None:
        y = y + b
    return activate(y.astype(F32), act)


def layer_norm(x, alpha, skip, gammas, betas, eps):
    """`LayerNorm2DWithSkipConnection` (backends/blas/encoder.h:29-78):
    LN(alpha * x + skip) over the last axis, biased variance, two passes."""
    v = x * F32(alpha)
    if skip is not None:
        v = v + skip
    v = v.astype(F32)
    mean = v.mean(axis=-1, keepdims=True, dtype=F32)
    diff = v - mean
    var = (diff * diff).mean(axis=-1, keepdims=True, dtype=F32)
    den = F32(1) / np.sqrt(var + F32(eps))
    return (betas + gammas * diff * den).astype(F32)


def softmax(x):
    """`SoftmaxActivation` (backends/shared/activation.cc:37-49)."""
    e = np.exp(x - x.max(axis=-1, keepdims=True))
    return (e / e.sum(axis=-1, keepdims=True, dtype=F32)).astype(F32)


def conv3x3(x, w, cout):
    """3x3 same-padded convolution on 8x8 boards.  The reference evaluates it with
    Winograd F(2x2,3x3) (backends/blas/winograd_convolution3.cc:47-57); this is
    the direct form of the same sum.  x: [N][Cin][8][8], w: [Cout][Cin][3][3]."""
    n, cin = x.shape[0], x.shape[1]
    xp = np.zeros((n, cin, 10, 10), F32)
    xp[:, :, 1:9, 1:9] = x
    cols = np.empty((n, cin, 9, 8, 8), F32)
    for ky in range(3):
        for kx in range(3):
            cols[:, :, ky * 3 + kx] = xp[:, :, ky:ky + 8, kx:kx + 8]
    cols = cols.reshape(n, cin * 9, 64)
    return np.matmul(w.reshape(cout, cin * 9)[None], cols).reshape(n, cout, 8, 8).astype(F32)


def conv1x1(x, w, cout):
    """`Convolution1::Forward` (backends/blas/convolution1.cc:31-89)."""
    n, cin = x.shape[0], x.shape[1]
    return np.matmul(w.reshape(cout, cin)[None], x.reshape(n, cin, 64)).reshape(n, cout, 8, 8).astype(F32)


def se_unit(x, conv_bias, skip, w1, b1, w2, b2, act):
    """`ApplySEUnit` (backends/blas/se_unit.cc:31-91): the convolution bias enters
    after pooling and again through sigmoid(scale) * bias."""
    n, c = x.shape[0], x.shape[1]
    k = b1.size
    pool = x.reshape(n, c, 64).mean(axis=2, dtype=F32) + conv_bias
    h = fc(pool, w1, b1, act, k)
    z = fc(h, w2, b2, ACT_NONE, 2 * c)
    gamma = F32(1) / (F32(1) + np.exp(-z[:, :c]))
    beta = z[:, c:] + gamma * conv_bias
    out = gamma[:, :, None, None] * x + skip + beta[:, :, None, None]
    return activate(out.astype(F32), act)


def encoder_layer(x, t, p, emb, heads, smolgen_act, ffn_act, alpha, eps, smolgen_w):
    """`BlasComputation::ForwardEncoderLayer` (backends/blas/network_blas.cc:271-471).
    x: [N][64][emb]; `p` is the tensor-name prefix of the layer."""
    n = x.shape[0]
    d_model = t[p + ".mha.q_b"].size
    dff = t[p + ".ffn.dense1_b"].size
    depth = d_model // heads
    bias = None
    if p + ".mha.smolgen.compress" in t:  # :300-339
        hc = t[p + ".mha.smolgen.compress"].size // emb
        hid = t[p + ".mha.smolgen.dense1_b"].size
        gen = t[p + ".mha.smolgen.dense2_b"].size
        c = fc(x.reshape(n * 64, emb), t[p + ".mha.smolgen.compress"], None, ACT_NONE, hc)
        h1 = fc(c.reshape(n, 64 * hc), t[p + ".mha.smolgen.dense1_w"], t[p + ".mha.smolgen.dense1_b"],
                smolgen_act, hid)
        h1 = layer_norm(h1, 1.0, None, t[p + ".mha.smolgen.ln1_gammas"], t[p + ".mha.smolgen.ln1_betas"], 1e-3)
        h2 = fc(h1, t[p + ".mha.smolgen.dense2_w"], t[p + ".mha.smolgen.dense2_b"], smolgen_act, gen)
        h2 = layer_norm(h2, 1.0, None, t[p + ".mha.smolgen.ln2_gammas"], t[p + ".mha.smolgen.ln2_betas"], 1e-3)
        bias = fc(h2.reshape(n * heads, gen // heads), smolgen_w, None, ACT_NONE, 4096)
        bias = bias.reshape(n, heads, 64, 64)
    xf = x.reshape(n * 64, emb)
    q = fc(xf, t[p + ".mha.q_w"], t[p + ".mha.q_b"], ACT_NONE, d_model).reshape(n, 64, heads, depth)
    k = fc(xf, t[p + ".mha.k_w"], t[p + ".mha.k_b"], ACT_NONE, d_model).reshape(n, 64, heads, depth)
    v = fc(xf, t[p + ".mha.v_w"], t[p + ".mha.v_b"], ACT_NONE, d_model).reshape(n, 64, heads, depth)
    scaling = F32(1.0) / np.sqrt(F32(depth))
    s = np.einsum("nqhd,nkhd->nhqk", q, k, dtype=F32) * scaling  # :357-393
    if bias is not None:
        s = s + bias
    pr = softmax(s.astype(F32))  # :395-406
    o = np.einsum("nhqk,nkhd->nqhd", pr, v, dtype=F32).reshape(n * 64, d_model)  # :414-439
    y = fc(o, t[p + ".mha.dense_w"], t[p + ".mha.dense_b"], ACT_NONE, emb)  # :441-445
    x1 = layer_norm(y, alpha, xf, t[p + ".ln1_gammas"], t[p + ".ln1_betas"], eps)  # :447-452
    f = fc(x1, t[p + ".ffn.dense1_w"], t[p + ".ffn.dense1_b"], ffn_act, dff)  # :454-458
    z = fc(f, t[p + ".ffn.dense2_w"], t[p + ".ffn.dense2_b"], ACT_NONE, t[p + ".ffn.dense2_b"].size)
    x2 = layer_norm(z, alpha, x1, t[p + ".ln2_gammas"], t[p + ".ln2_betas"], eps)  # :465-470
    return x2.reshape(n, 64, emb)


def forward(meta, t, masks, values, mlh=True, chunk=256):
    """`BlasComputation::ComputeBlocking` (backends/blas/network_blas.cc:473-971).

    Returns dict(policy=[N][1858] raw logits, q=[N], d=[N], m=[N]) with the
    accessor semantics of GetQVal/GetDVal/GetMVal (:85-116)."""
    masks = np.asarray(masks, np.uint64).reshape(-1, 112)
    values = np.asarray(values, F32).reshape(-1, 112)
    outs = [_forward_chunk(meta, t, masks[i:i + chunk], values[i:i + chunk], mlh)
            for i in range(0, masks.shape[0], chunk)]
    if not outs:
        z = np.zeros(0, F32)
        return dict(policy=np.zeros((0, 1858), F32), q=z, d=z, m=z)
    return {k: np.concatenate([o[k] for o in outs]) for k in outs[0]}


def _forward_chunk(meta, t, masks, values, mlh):
    tb = _tables()
    n = masks.shape[0]
    act = meta["default_activation"]
    attn_body = meta["network"] in (6, 7)
    attn_policy = meta["policy"] == 3
    conv_policy = meta["policy"] == 2
    wdl = meta["value"] == 2
    moves_left = meta["moves_left"] == 1 and mlh
    pe_dense = meta["input_embedding"] == 2
    planes = expand_planes(masks, values)  # [n][112][64]
    res_blocks = sum(1 for k in t if k.startswith("residual.") and k.endswith(".conv1.weights"))

    flow = None  # NCHW activations of the residual tower
    if res_blocks > 0:  # :564-601
        c = t["input.biases"].size
        flow = conv3x3(planes.reshape(n, 112, 8, 8), t["input.weights"], c)
        flow = activate(flow + t["input.biases"][None, :, None, None], act)
        for i in range(res_blocks):
            p = "residual.%d" % i
            a = conv3x3(flow, t[p + ".conv1.weights"], c)
            a = activate(a + t[p + ".conv1.biases"][None, :, None, None], act)
            b = conv3x3(a, t[p + ".conv2.weights"], c)
            if p + ".se.w1" in t:
                flow = se_unit(b, t[p + ".conv2.biases"], flow, t[p + ".se.w1"], t[p + ".se.b1"],
                               t[p + ".se.w2"], t[p + ".se.b2"], act)
            else:
                flow = activate(b + t[p + ".conv2.biases"][None, :, None, None] + flow, act)

    x = None  # token-major activations of the attention body
    if attn_body:  # :603-721
        emb = t["ip_emb_b"].size
        if res_blocks == 0:
            tokens = planes.transpose(0, 2, 1)  # NCHW -> NHWC, [n][64][112]
            if pe_dense:  # :612-628
                enc_ch = t["ip_emb_preproc_b"].size // 64
                pre_in = tokens[:, :, :12].reshape(n, 64 * 12)
                pe = fc(pre_in, t["ip_emb_preproc_w"], t["ip_emb_preproc_b"], ACT_NONE, 64 * enc_ch)
                tokens = np.concatenate([tokens, pe.reshape(n, 64, enc_ch)], axis=2)
            else:  # :645-650
                pe = np.broadcast_to(tb.pos_encoding()[None], (n, 64, 64))
                tokens = np.concatenate([tokens, pe], axis=2)
        else:
            tokens = flow.reshape(n, -1, 64).transpose(0, 2, 1)
        in_size = tokens.shape[2]
        x = fc(tokens.reshape(n * 64, in_size).astype(F32), t["ip_emb_w"], t["ip_emb_b"], act, emb)
        if pe_dense:  # :662-667
            x = layer_norm(x, 1.0, None, t["ip_emb_ln_gammas"], t["ip_emb_ln_betas"], 1e-3)
        x = x.reshape(n, 64, emb)
        if "ip_mult_gate" in t and "ip_add_gate" in t:  # :669-682, gates stored [emb][64]
            x = x * t["ip_mult_gate"].reshape(emb, 64).T[None] + t["ip_add_gate"].reshape(emb, 64).T[None]
            x = x.astype(F32)
        layers = sum(1 for k in t if k.startswith("encoder.") and k.endswith(".mha.q_w"))
        alpha = F32(np.power(2.0 * layers, -0.25))  # :684
        if pe_dense:  # :687-712
            dff = t["ip_emb_ffn.dense1_b"].size
            xf = x.reshape(n * 64, emb)
            f = fc(xf, t["ip_emb_ffn.dense1_w"], t["ip_emb_ffn.dense1_b"], meta["ffn_activation"], dff)
            z = fc(f, t["ip_emb_ffn.dense2_w"], t["ip_emb_ffn.dense2_b"], ACT_NONE, emb)
            x = layer_norm(z, alpha, xf, t["ip_emb_ffn_ln_gammas"], t["ip_emb_ffn_ln_betas"], 1e-3)
            x = x.reshape(n, 64, emb)
        for i in range(layers):  # :715-720
            x = encoder_layer(x, t, "encoder.%d" % i, emb, meta["headcount"], meta["smolgen_activation"],
                              meta["ffn_activation"], alpha, 1e-3 if pe_dense else 1e-6,
                              t.get("smolgen_w"))

    # ---- value head (:725-772) ----
    vh = t["value.ip1_val_b"].size
    if attn_body:
        vp = t["value.ip_val_b"].size
        hv = fc(x.reshape(n * 64, -1), t["value.ip_val_w"], t["value.ip_val_b"], act, vp).reshape(n, 64 * vp)
    else:
        vp = t["value.value.biases"].size
        hv = conv1x1(flow, t["value.value.weights"], vp) + t["value.value.biases"][None, :, None, None]
        hv = activate(hv, act).reshape(n, vp * 64)
    hv = fc(hv, t["value.ip1_val_w"], t["value.ip1_val_b"], act, vh)
    if wdl:
        w3 = softmax(fc(hv, t["value.ip2_val_w"], t["value.ip2_val_b"], ACT_NONE, 3))
        q, d = (w3[:, 0] - w3[:, 2]).astype(F32), w3[:, 1].astype(F32)
    else:
        win = hv.astype(np.float64) @ t["value.ip2_val_w"].astype(np.float64) + float(t["value.ip2_val_b"][0])
        q, d = np.tanh(win).astype(F32), np.zeros(n, F32)

    # ---- moves-left head (:775-803) ----
    m = np.zeros(n, F32)
    if moves_left:
        mh = t["ip1_mov_b"].size
        if attn_body:
            mp = t["ip_mov_b"].size
            hm = fc(x.reshape(n * 64, -1), t["ip_mov_w"], t["ip_mov_b"], act, mp).reshape(n, 64 * mp)
        else:
            mp = t["moves_left.biases"].size
            hm = conv1x1(flow, t["moves_left.weights"], mp) + t["moves_left.biases"][None, :, None, None]
            hm = activate(hm, act).reshape(n, mp * 64)
        hm = fc(hm, t["ip1_mov_w"], t["ip1_mov_b"], act, mh)
        m = fc(hm, t["ip2_mov_w"], t["ip2_mov_b"], ACT_RELU, 1).reshape(n)

    # ---- policy head (:806-968) ----
    if attn_policy:
        if attn_body:
            src, pol_act, in_ch = x.reshape(n * 64, -1), act, x.shape[2]
        else:
            in_ch = flow.shape[1]
            src, pol_act = flow.reshape(n, in_ch, 64).transpose(0, 2, 1).reshape(n * 64, in_ch), ACT_SELU
        pe_sz = t["policy.ip_pol_b"].size
        p0 = fc(src, t["policy.ip_pol_w"], t["policy.ip_pol_b"], pol_act, pe_sz).reshape(n, 64, pe_sz)
        n_pol_enc = sum(1 for k in t if k.startswith("policy.pol_encoder.") and k.endswith(".mha.q_w"))
        for i in range(n_pol_enc):  # :832-838
            p0 = encoder_layer(p0, t, "policy.pol_encoder.%d" % i, pe_sz, meta["pol_headcount"],
                               meta["smolgen_activation"] if attn_body else ACT_NONE,
                               meta["ffn_activation"] if attn_body else ACT_SELU, 1.0, 1e-6,
                               t.get("smolgen_w"))
        dm = t["policy.ip2_pol_b"].size
        pq = fc(p0.reshape(n * 64, pe_sz), t["policy.ip2_pol_w"], t["policy.ip2_pol_b"], ACT_NONE, dm)
        pk = fc(p0.reshape(n * 64, pe_sz), t["policy.ip3_pol_w"], t["policy.ip3_pol_b"], ACT_NONE, dm)
        pq, pk = pq.reshape(n, 64, dm), pk.reshape(n, 64, dm)
        logits = np.matmul(pq, pk.transpose(0, 2, 1)) * (F32(1.0) / np.sqrt(F32(dm)))  # :850-872
        off = np.einsum("njk,ik->nij", pk[:, 56:64, :], t["policy.ip4_pol_w"].reshape(4, dm))  # :873-887
        off = off.astype(F32)
        off[:, :3, :] += off[:, 3:4, :]
        promo = logits[:, 48:56, 56:64][:, :, :, None] + off[:, :3, :].transpose(0, 2, 1)[:, None, :, :]
        raw = np.concatenate([logits.reshape(n, 4096), promo.reshape(n, 192)], axis=1).astype(F32)
        policy = _gather(raw, tb.attn_policy_map())  # :904-914
    elif conv_policy:  # :915-942
        c = flow.shape[1]
        pp = t["policy.policy.biases"].size
        a = conv3x3(flow, t["policy.policy1.weights"], c)
        a = activate(a + t["policy.policy1.biases"][None, :, None, None], act)
        b = conv3x3(a, t["policy.policy.weights"], pp) + t["policy.policy.biases"][None, :, None, None]
        policy = _gather(b.reshape(n, pp * 64)[:, :73 * 64].astype(F32), tb.conv_policy_map())
    else:  # :944-968
        pp = t["policy.policy.biases"].size
        a = conv1x1(flow, t["policy.policy.weights"], pp) + t["policy.policy.biases"][None, :, None, None]
        a = activate(a, act).reshape(n, pp * 64)
        policy = fc(a, t["policy.ip_pol_w"], t["policy.ip_pol_b"], ACT_NONE, 1858)
    return dict(policy=policy.astype(F32), q=q, d=d, m=m.astype(F32))


def _gather(raw, pmap):
    out = np.zeros((raw.shape[0], 1858), F32)
    valid = pmap >= 0
    out[:, pmap[valid]] = raw[:, valid]
    return out


def fast_exp(x):
    """`FastExp` / `FastExp2` (utils/fastmath.h:59-86) on float32 arrays, operation by operation."""
    a = (F32(1.442695040) * np.asarray(x, F32)).astype(F32)
    neg = a < 0
    e = np.where(neg, (a - F32(1)).astype(F32), a).astype(np.int32)  # C cast truncates toward zero
    out = (a - e.astype(F32)).astype(F32)
    out = (F32(1) + out * (F32(0.6602339) + F32(0.33976606) * out).astype(F32)).astype(F32)
    bits = out.view(np.int32) + (e.astype(np.uint32) << np.uint32(23)).astype(np.int32)
    res = bits.view(F32)
    return np.where(a < F32(-126), F32(0), res).astype(F32)


def softmax_policy(policy_row, move_ids, inv_temperature=1.0):
    """`NetworkAsBackendComputation::SoftmaxPolicy` (neural/wrapper.cc:135-156): legal-move softmax with FastExp
    and a sequentially accumulated total."""
    v = np.asarray(policy_row, F32)[np.asarray(move_ids, np.int64)]
    if v.size == 0:
        return v
    e = fast_exp(((v - v.max()) * F32(inv_temperature)).astype(F32))
    total = F32(0)
    for t in e:
        total = F32(total + t)
    scale = F32(1) / total if total > 0 else F32(1)
    return (e * scale).astype(F32)


def legal_softmax(policy_row, legal_indices):
    """Softmax over the legal moves only, temperature 1 (what the caller does with
    GetPVal, neural/wrapper.cc:135-156)."""
    x = policy_row[legal_indices].astype(F32)
    e = np.exp(x - x.max())
    return e / e.sum()
