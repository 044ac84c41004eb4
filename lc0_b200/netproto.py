"""Reader and writer for lc0 weight files (`net.proto`, optionally gzipped).

The schema below restates the message layout of the reference's
proto/net.proto:31-411 (field numbers and wire types only); the wire codec is a
small self-contained proto2 implementation, so no protobuf runtime or generated
code is needed.  Messages are plain dicts: scalar fields map to Python values,
sub-messages to dicts, repeated fields to lists.  A `Layer` keeps its raw
`params` bytes; decoding to floats follows the reference's LayerAdapter
(utils/weights_adapter.cc:38-62) in :func:`layer_to_array`.
"""
import gzip
import struct

import numpy as np

WEIGHT_MAGIC = 0x1C0  # neural/loader.cc: kWeightMagic

# Layer.Encoding (proto/net.proto:42-48)
LINEAR16, FLOAT16, BFLOAT16, FLOAT32 = 1, 2, 3, 4

# ---- schema: message -> {field_number: (name, type, repeated)} ----------------
# type is one of: uint32, enum, float, fixed32, bytes, string, or a message name.
_L = "Layer"
SCHEMA = {
    "EngineVersion": {1: ("major", "uint32", 0), 2: ("minor", "uint32", 0), 3: ("patch", "uint32", 0)},
    "Layer": {1: ("min_val", "float", 0), 2: ("max_val", "float", 0), 3: ("params", "bytes", 0),
              4: ("encoding", "enum", 0), 5: ("dims", "uint32", 1)},
    "ConvBlock": {1: ("weights", _L, 0), 2: ("biases", _L, 0), 3: ("bn_means", _L, 0),
                  4: ("bn_stddivs", _L, 0), 5: ("bn_gammas", _L, 0), 6: ("bn_betas", _L, 0)},
    "SEunit": {1: ("w1", _L, 0), 2: ("b1", _L, 0), 3: ("w2", _L, 0), 4: ("b2", _L, 0)},
    "Residual": {1: ("conv1", "ConvBlock", 0), 2: ("conv2", "ConvBlock", 0), 3: ("se", "SEunit", 0)},
    "Smolgen": {1: ("compress", _L, 0), 2: ("dense1_w", _L, 0), 3: ("dense1_b", _L, 0),
                4: ("ln1_gammas", _L, 0), 5: ("ln1_betas", _L, 0), 6: ("dense2_w", _L, 0),
                7: ("dense2_b", _L, 0), 8: ("ln2_gammas", _L, 0), 9: ("ln2_betas", _L, 0)},
    "MHA": {1: ("q_w", _L, 0), 2: ("q_b", _L, 0), 3: ("k_w", _L, 0), 4: ("k_b", _L, 0),
            5: ("v_w", _L, 0), 6: ("v_b", _L, 0), 7: ("dense_w", _L, 0), 8: ("dense_b", _L, 0),
            9: ("smolgen", "Smolgen", 0), 10: ("rpe_q", _L, 0), 11: ("rpe_k", _L, 0),
            12: ("rpe_v", _L, 0)},
    "FFN": {1: ("dense1_w", _L, 0), 2: ("dense1_b", _L, 0), 3: ("dense2_w", _L, 0),
            4: ("dense2_b", _L, 0)},
    "EncoderLayer": {1: ("mha", "MHA", 0), 2: ("ln1_gammas", _L, 0), 3: ("ln1_betas", _L, 0),
                     4: ("ffn", "FFN", 0), 5: ("ln2_gammas", _L, 0), 6: ("ln2_betas", _L, 0)},
    "PolicyHead": {1: ("ip_pol_w", _L, 0), 2: ("ip_pol_b", _L, 0), 3: ("ip2_pol_w", _L, 0),
                   4: ("ip2_pol_b", _L, 0), 5: ("ip3_pol_w", _L, 0), 6: ("ip3_pol_b", _L, 0),
                   7: ("ip4_pol_w", _L, 0), 8: ("pol_encoder", "EncoderLayer", 1),
                   9: ("pol_headcount", "uint32", 0), 10: ("policy1", "ConvBlock", 0),
                   11: ("policy", "ConvBlock", 0)},
    "ValueHead": {1: ("ip_val_w", _L, 0), 2: ("ip_val_b", _L, 0), 3: ("ip1_val_w", _L, 0),
                  4: ("ip1_val_b", _L, 0), 5: ("ip2_val_w", _L, 0), 6: ("ip2_val_b", _L, 0),
                  7: ("ip_val_err_w", _L, 0), 8: ("ip_val_err_b", _L, 0), 9: ("ip_val_cat_w", _L, 0),
                  10: ("ip_val_cat_b", _L, 0), 11: ("value", "ConvBlock", 0)},
    "PolicyHeadMap": {1: ("key", "string", 0), 2: ("value", "PolicyHead", 0)},
    "PolicyHeads": {1: ("ip_pol_w", _L, 0), 2: ("ip_pol_b", _L, 0), 3: ("vanilla", "PolicyHead", 0),
                    4: ("optimistic_st", "PolicyHead", 0), 5: ("soft", "PolicyHead", 0),
                    6: ("opponent", "PolicyHead", 0), 7: ("policy_head_map", "PolicyHeadMap", 1)},
    "ValueHeadMap": {1: ("key", "string", 0), 2: ("value", "ValueHead", 0)},
    "ValueHeads": {1: ("winner", "ValueHead", 0), 2: ("q", "ValueHead", 0), 3: ("st", "ValueHead", 0),
                   4: ("value_head_map", "ValueHeadMap", 1)},
    "Weights": {
        1: ("input", "ConvBlock", 0), 2: ("residual", "Residual", 1),
        37: ("ip_emb_preproc_w", _L, 0), 38: ("ip_emb_preproc_b", _L, 0),
        25: ("ip_emb_w", _L, 0), 26: ("ip_emb_b", _L, 0),
        39: ("ip_emb_ln_gammas", _L, 0), 40: ("ip_emb_ln_betas", _L, 0),
        33: ("ip_mult_gate", _L, 0), 34: ("ip_add_gate", _L, 0),
        41: ("ip_emb_ffn", "FFN", 0), 42: ("ip_emb_ffn_ln_gammas", _L, 0),
        43: ("ip_emb_ffn_ln_betas", _L, 0),
        27: ("encoder", "EncoderLayer", 1), 28: ("headcount", "uint32", 0),
        21: ("pol_encoder", "EncoderLayer", 1), 24: ("pol_headcount", "uint32", 0),
        11: ("policy1", "ConvBlock", 0), 3: ("policy", "ConvBlock", 0),
        4: ("ip_pol_w", _L, 0), 5: ("ip_pol_b", _L, 0), 17: ("ip2_pol_w", _L, 0),
        18: ("ip2_pol_b", _L, 0), 19: ("ip3_pol_w", _L, 0), 20: ("ip3_pol_b", _L, 0),
        22: ("ip4_pol_w", _L, 0),
        6: ("value", "ConvBlock", 0), 29: ("ip_val_w", _L, 0), 30: ("ip_val_b", _L, 0),
        7: ("ip1_val_w", _L, 0), 8: ("ip1_val_b", _L, 0), 9: ("ip2_val_w", _L, 0),
        10: ("ip2_val_b", _L, 0),
        44: ("value_heads", "ValueHeads", 0), 45: ("policy_heads", "PolicyHeads", 0),
        12: ("moves_left", "ConvBlock", 0), 31: ("ip_mov_w", _L, 0), 32: ("ip_mov_b", _L, 0),
        13: ("ip1_mov_w", _L, 0), 14: ("ip1_mov_b", _L, 0), 15: ("ip2_mov_w", _L, 0),
        16: ("ip2_mov_b", _L, 0),
        35: ("smolgen_w", _L, 0), 36: ("smolgen_b", _L, 0)},
    "TrainingParams": {1: ("training_steps", "uint32", 0), 2: ("learning_rate", "float", 0),
                       3: ("mse_loss", "float", 0), 4: ("policy_loss", "float", 0),
                       5: ("accuracy", "float", 0), 6: ("lc0_params", "string", 0)},
    "NetworkFormat": {1: ("input", "enum", 0), 2: ("output", "enum", 0), 3: ("network", "enum", 0),
                      4: ("policy", "enum", 0), 5: ("value", "enum", 0), 6: ("moves_left", "enum", 0),
                      7: ("default_activation", "enum", 0), 8: ("smolgen_activation", "enum", 0),
                      9: ("ffn_activation", "enum", 0), 10: ("input_embedding", "enum", 0)},
    "Format": {1: ("weights_encoding", "enum", 0), 2: ("network_format", "NetworkFormat", 0)},
    "OnnxModel": {1: ("model", "bytes", 0), 2: ("data_type", "enum", 0), 3: ("input_planes", "string", 0),
                  4: ("output_value", "string", 0), 5: ("output_wdl", "string", 0),
                  6: ("output_policy", "string", 0), 7: ("output_mlh", "string", 0)},
    "Net": {1: ("magic", "fixed32", 0), 2: ("license", "string", 0), 3: ("min_version", "EngineVersion", 0),
            4: ("format", "Format", 0), 5: ("training_params", "TrainingParams", 0),
            10: ("weights", "Weights", 0), 11: ("onnx_model", "OnnxModel", 0)},
}
_BY_NAME = {m: {v[0]: (k, v[1], v[2]) for k, v in f.items()} for m, f in SCHEMA.items()}


# NetworkFormat enum values (proto/net.proto:275-367) used by this package.
class NF:
    INPUT_CLASSICAL_112_PLANE = 1
    INPUT_112_WITH_CASTLING_PLANE = 2
    OUTPUT_CLASSICAL, OUTPUT_WDL = 1, 2
    NETWORK_CLASSICAL, NETWORK_SE = 1, 2
    NETWORK_CLASSICAL_WITH_HEADFORMAT, NETWORK_SE_WITH_HEADFORMAT = 3, 4
    NETWORK_ONNX = 5
    NETWORK_ATTENTIONBODY_WITH_HEADFORMAT = 6
    NETWORK_ATTENTIONBODY_WITH_MULTIHEADFORMAT = 7
    NETWORK_AB_LEGACY_WITH_MULTIHEADFORMAT = 134
    POLICY_CLASSICAL, POLICY_CONVOLUTION, POLICY_ATTENTION = 1, 2, 3
    VALUE_CLASSICAL, VALUE_WDL, VALUE_PARAM = 1, 2, 3
    MOVES_LEFT_NONE, MOVES_LEFT_V1 = 0, 1
    DEFAULT_ACTIVATION_RELU, DEFAULT_ACTIVATION_MISH = 0, 1
    ACTIVATION_DEFAULT, ACTIVATION_MISH, ACTIVATION_RELU, ACTIVATION_NONE = 0, 1, 2, 3
    ACTIVATION_TANH, ACTIVATION_SIGMOID, ACTIVATION_SELU, ACTIVATION_SWISH = 4, 5, 6, 7
    ACTIVATION_RELU_2, ACTIVATION_SOFTMAX = 8, 9
    INPUT_EMBEDDING_NONE, INPUT_EMBEDDING_PE_MAP, INPUT_EMBEDDING_PE_DENSE = 0, 1, 2


# ---- wire codec -----------------------------------------------------------------
def _varint(v):
    out = bytearray()
    v &= (1 << 64) - 1
    while True:
        b = v & 0x7F
        v >>= 7
        if v:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _read_varint(buf, pos):
    shift = 0
    val = 0
    while True:
        if pos >= len(buf):
            raise ValueError("truncated varint")
        b = buf[pos]
        pos += 1
        val |= (b & 0x7F) << shift
        if not b & 0x80:
            return val, pos
        shift += 7
        if shift > 70:
            raise ValueError("varint too long")


def encode(msg_name, msg):
    """Serialise dict `msg` as proto2 message `msg_name`."""
    fields = _BY_NAME[msg_name]
    out = []
    for name, val in msg.items():
        if val is None:
            continue
        num, typ, rep = fields[name]
        vals = val if rep else [val]
        for v in vals:
            if typ in ("uint32", "enum"):
                out.append(_varint(num << 3 | 0) + _varint(int(v)))
            elif typ == "float":
                out.append(_varint(num << 3 | 5) + struct.pack("<f", v))
            elif typ == "fixed32":
                out.append(_varint(num << 3 | 5) + struct.pack("<I", v))
            elif typ in ("bytes", "string"):
                b = v.encode() if isinstance(v, str) else bytes(v)
                out.append(_varint(num << 3 | 2) + _varint(len(b)) + b)
            else:
                b = encode(typ, v)
                out.append(_varint(num << 3 | 2) + _varint(len(b)) + b)
    return b"".join(out)


def decode(msg_name, buf):
    """Parse bytes `buf` as proto2 message `msg_name`; unknown fields are skipped."""
    fields = SCHEMA[msg_name]
    buf = memoryview(buf)
    pos = 0
    msg = {}
    n = len(buf)
    while pos < n:
        key, pos = _read_varint(buf, pos)
        num, wt = key >> 3, key & 7
        if wt == 0:
            raw, pos = _read_varint(buf, pos)
        elif wt == 5:
            if pos + 4 > n:
                raise ValueError("truncated fixed32")
            raw = bytes(buf[pos:pos + 4])
            pos += 4
        elif wt == 1:
            if pos + 8 > n:
                raise ValueError("truncated fixed64")
            raw = bytes(buf[pos:pos + 8])
            pos += 8
        elif wt == 2:
            ln, pos = _read_varint(buf, pos)
            if pos + ln > n:
                raise ValueError("truncated length-delimited field")
            raw = buf[pos:pos + ln]
            pos += ln
        else:
            raise ValueError("unsupported wire type %d" % wt)
        if num not in fields:
            continue
        name, typ, rep = fields[num]
        if typ in ("uint32", "enum"):
            if wt == 2:  # packed repeated
                vals, p2 = [], 0
                while p2 < len(raw):
                    v, p2 = _read_varint(raw, p2)
                    vals.append(v)
                msg.setdefault(name, []).extend(vals)
                continue
            val = raw
        elif typ == "float":
            val = struct.unpack("<f", raw)[0]
        elif typ == "fixed32":
            val = struct.unpack("<I", raw)[0]
        elif typ == "bytes":
            val = bytes(raw)
        elif typ == "string":
            val = bytes(raw).decode("utf-8", "replace")
        else:
            val = decode(typ, raw)
        if rep:
            msg.setdefault(name, []).append(val)
        else:
            msg[name] = val
    return msg


# ---- Layer <-> numpy --------------------------------------------------------------
def array_to_layer(arr, encoding=FLOAT32):
    """Pack a float array into a `Layer` dict with the given per-layer encoding."""
    a = np.ascontiguousarray(arr, dtype=np.float32).reshape(-1)
    if encoding == FLOAT32:
        return {"params": a.astype("<f4").tobytes(), "encoding": FLOAT32}
    if encoding == FLOAT16:
        return {"params": a.astype("<f2").tobytes(), "encoding": FLOAT16}
    if encoding == BFLOAT16:
        u = a.view(np.uint32)
        return {"params": (u >> 16).astype("<u2").tobytes(), "encoding": BFLOAT16}
    if encoding == LINEAR16:
        lo, hi = (float(a.min()), float(a.max())) if a.size else (0.0, 0.0)
        span = hi - lo if hi > lo else 1.0
        q = np.clip(np.rint((a - lo) / span * 65535.0), 0, 65535).astype("<u2")
        return {"min_val": lo, "max_val": hi, "params": q.tobytes(), "encoding": LINEAR16}
    raise ValueError("unknown layer encoding %r" % (encoding,))


def layer_to_array(layer):
    """Decode a `Layer` dict to float32 (utils/weights_adapter.cc:38-62, :64-73:
    a layer without an `encoding` field is LINEAR16)."""
    if not layer:
        return np.zeros(0, np.float32)
    enc = layer.get("encoding", LINEAR16)
    raw = layer.get("params", b"")
    if enc == FLOAT32:
        return np.frombuffer(raw, "<f4").astype(np.float32)
    if enc == FLOAT16:
        return np.frombuffer(raw, "<f2").astype(np.float32)
    if enc == BFLOAT16:
        return (np.frombuffer(raw, "<u2").astype(np.uint32) << 16).view(np.float32)
    if enc == LINEAR16:
        theta = np.frombuffer(raw, "<u2").astype(np.float32) / np.float32(65535.0)
        lo = np.float32(layer.get("min_val", 0.0))
        hi = np.float32(layer.get("max_val", 0.0))
        return (lo * (np.float32(1) - theta) + hi * theta).astype(np.float32)
    raise ValueError("Unknown layer encoding %r" % (enc,))


# ---- files -------------------------------------------------------------------------
def write_net(path, net, compress=True):
    data = encode("Net", net)
    if compress:
        with gzip.GzipFile(path, "wb", compresslevel=1, mtime=0) as f:
            f.write(data)
    else:
        with open(path, "wb") as f:
            f.write(data)


def read_net_bytes(path):
    with open(path, "rb") as f:
        head = f.read(2)
    if head == b"\x1f\x8b":
        with gzip.open(path, "rb") as f:
            return f.read()
    with open(path, "rb") as f:
        return f.read()


def _version_int(major, minor, patch):
    return major * 1000000 + minor * 1000 + patch  # version.cc:29-31


LC0_VERSION = (0, 33, 0)


def fix_older_format(net):
    """Format fix-ups the reference applies after parsing (neural/loader.cc:108-158)."""
    fmt = net.setdefault("format", {})
    has_nf = "network_format" in fmt
    nf = fmt.setdefault("network_format", {})
    network = nf.get("network", 0)
    w = net.get("weights", {})
    if not has_nf:
        nf.update(input=NF.INPUT_CLASSICAL_112_PLANE, output=NF.OUTPUT_CLASSICAL,
                  network=NF.NETWORK_CLASSICAL_WITH_HEADFORMAT, value=NF.VALUE_CLASSICAL,
                  policy=NF.POLICY_CLASSICAL)
    elif network == NF.NETWORK_CLASSICAL:
        nf.update(network=NF.NETWORK_CLASSICAL_WITH_HEADFORMAT, value=NF.VALUE_CLASSICAL,
                  policy=NF.POLICY_CLASSICAL)
    elif network == NF.NETWORK_SE:
        nf.update(network=NF.NETWORK_SE_WITH_HEADFORMAT, value=NF.VALUE_CLASSICAL,
                  policy=NF.POLICY_CLASSICAL)
    elif network == NF.NETWORK_SE_WITH_HEADFORMAT and len(w.get("encoder", [])) > 0:
        nf["network"] = NF.NETWORK_ATTENTIONBODY_WITH_HEADFORMAT
        if "smolgen_w" in w:
            nf["ffn_activation"] = NF.ACTIVATION_RELU_2
            nf["smolgen_activation"] = NF.ACTIVATION_SWISH
    elif network == NF.NETWORK_AB_LEGACY_WITH_MULTIHEADFORMAT:
        nf["network"] = NF.NETWORK_ATTENTIONBODY_WITH_MULTIHEADFORMAT
    if nf.get("network", 0) == NF.NETWORK_ATTENTIONBODY_WITH_HEADFORMAT:
        if "policy_heads" in w and "value_heads" in w:
            nf["network"] = NF.NETWORK_ATTENTIONBODY_WITH_MULTIHEADFORMAT
            nf["input_embedding"] = NF.INPUT_EMBEDDING_PE_DENSE
        if "input_embedding" not in nf:
            nf["input_embedding"] = NF.INPUT_EMBEDDING_PE_MAP
    return net


def parse_net(data):
    """Parse + validate like the reference loader (neural/loader.cc:160-191)."""
    if len(data) < 2:
        raise ValueError("Invalid weight file: too small.")
    if data[:2] in (b"1\n", b"2\n"):
        raise ValueError("Invalid weight file: text formats are no longer supported.")
    net = decode("Net", data)
    if net.get("magic", 0) != WEIGHT_MAGIC:
        raise ValueError("Invalid weight file: bad header.")
    mv = net.get("min_version", {})
    net_ver = _version_int(mv.get("major", 0), mv.get("minor", 0), mv.get("patch", 0))
    fix_older_format(net)
    if net_ver != 0x5C99973 and net_ver > _version_int(*LC0_VERSION):
        raise ValueError("Invalid weight file: lc0 version >= %d.%d.%d required." %
                         (mv.get("major", 0), mv.get("minor", 0), mv.get("patch", 0)))
    if "weights" in net and net["format"].get("weights_encoding", 0) != 1 and \
            net_ver < _version_int(0, 33, 0):
        raise ValueError("Invalid weight file: unsupported encoding.")
    return net


def load_net(path):
    return parse_net(read_net_bytes(path))
