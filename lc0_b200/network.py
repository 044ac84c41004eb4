"""Host-side mirror of lc0's backend plug-in interface over the C ABI.

`Network` / `NetworkComputation` follow lczero::Network / lczero::NetworkComputation
(src/neural/network.h:56-126): same method names (snake_case of AddInput, ComputeBlocking,
GetBatchSize, GetQVal, GetDVal, GetMVal, GetPVal), same argument meaning, and the
error behaviour of the reference's backends (unknown head names, unsupported formats, bad
GPU ids and unknown options raise).  `create_network` plays the role of the factory lambda
registered by REGISTER_NETWORK (src/neural/factory.h:111-142): weights file + option
string in, network out.
"""
import ctypes

import numpy as np

from . import _lib, netproto, weights as _weights

_KNOWN_OPTIONS = {"gpu", "max_batch", "precision", "slots", "mlh", "policy_head", "value_head",
                  "tensor_cores", "graph_capture", "fold_ln", "merge_compress", "split_last_wave", "fused_se", "winograd",
                  "side_stream", "dependent_launch", "tower"}


def parse_options(opts):
    """Parse a `key=value,key=value` backend-options string (the flat subset of
    lc0's OptionsDict syntax, src/utils/optionsdict.cc:238-279). Unknown keys raise,
    like OptionsDict::CheckAllOptionsRead (src/utils/optionsdict.cc:331-341)."""
    if isinstance(opts, dict):
        d = dict(opts)
    else:
        d = {}
        for part in filter(None, (p.strip() for p in (opts or "").split(","))):
            if "=" not in part:
                raise ValueError("Bad backend option '%s' (expected key=value)" % part)
            k, v = part.split("=", 1)
            d[k.strip()] = v.strip()
    for k in d:
        if k not in _KNOWN_OPTIONS:
            raise ValueError("Unknown backend option: %s" % k)
    return d


def _as_bool(v):
    return str(v).lower() not in ("0", "false", "no", "off")


def option_flags(opts):
    """b200_net_options.flags from the boolean options (all default to on)."""
    flags = 0
    for key, bit in (("tensor_cores", _lib.FLAG_NO_TENSOR_CORES), ("graph_capture", _lib.FLAG_NO_GRAPHS),
                     ("fold_ln", _lib.FLAG_NO_LN_FOLD), ("merge_compress", _lib.FLAG_NO_MERGED_COMPRESS),
                     ("split_last_wave", _lib.FLAG_NO_SPLIT_LAST_WAVE), ("fused_se", _lib.FLAG_NO_FUSED_SE), ("side_stream", _lib.FLAG_NO_SIDE_STREAM),
                     ("dependent_launch", _lib.FLAG_NO_DEPENDENT_LAUNCH)):
        if not _as_bool(opts.get(key, True)):
            flags |= bit
    if _as_bool(opts.get("winograd", False)):
        flags |= _lib.FLAG_WINOGRAD
    if not _as_bool(opts.get("tower", True)):
        flags |= _lib.FLAG_NO_TOWER_KERNEL
    return flags


class NetworkComputation:
    """One batch: add_input x n, compute_blocking, then read results (single use)."""

    def __init__(self, network):
        self._lib = _lib.load()
        self._net = network
        h = ctypes.c_void_p()
        _lib.check(self._lib.b200_comp_create(network._handle, ctypes.byref(h)))
        self._h = h

    def add_input(self, masks, values):
        """AddInput: 112 plane masks (uint64) and 112 plane values (float32)."""
        m = np.ascontiguousarray(masks, np.uint64).reshape(-1)
        v = np.ascontiguousarray(values, np.float32).reshape(-1)
        if m.size != 112 or v.size != 112:
            raise ValueError("add_input expects 112 masks and 112 values")
        _lib.check(self._lib.b200_comp_add_input(self._h, m.ctypes.data, v.ctypes.data))

    def add_input_with_moves(self, masks, values, move_ids):
        """AddInput plus the policy indices of the position's legal moves (MoveToNNIndex of each move); the
        legal-move softmax then runs on the device (see `legal_policy`)."""
        m = np.ascontiguousarray(masks, np.uint64).reshape(-1)
        v = np.ascontiguousarray(values, np.float32).reshape(-1)
        ids = np.ascontiguousarray(move_ids, np.uint16).reshape(-1)
        if m.size != 112 or v.size != 112:
            raise ValueError("add_input expects 112 masks and 112 values")
        _lib.check(self._lib.b200_comp_add_input_with_moves(self._h, m.ctypes.data, v.ctypes.data, ids.ctypes.data,
                                                            ids.size))

    def add_inputs_with_moves(self, masks, values, move_ids, n_moves):
        """Batch form: move_ids [n][256] (rows padded), n_moves [n]."""
        m = np.ascontiguousarray(masks, np.uint64).reshape(-1, 112)
        v = np.ascontiguousarray(values, np.float32).reshape(-1, 112)
        ids = np.ascontiguousarray(move_ids, np.uint16).reshape(-1, 256)
        cnt = np.ascontiguousarray(n_moves, np.int32).reshape(-1)
        if not (m.shape[0] == v.shape[0] == ids.shape[0] == cnt.shape[0]):
            raise ValueError("masks, values, move_ids and n_moves must describe the same number of positions")
        _lib.check(self._lib.b200_comp_add_inputs_with_moves(self._h, m.ctypes.data, v.ctypes.data, ids.ctypes.data,
                                                             cnt.ctypes.data, m.shape[0]))

    def set_encoding(self, input_format=0, fill_empty_history=_lib.FILL_FEN_ONLY):
        """Input format (0: the network's) and FillEmptyHistory policy of the device-side position encoder."""
        _lib.check(self._lib.b200_comp_set_encoding(self._h, int(input_format), int(fill_empty_history)))

    def add_position(self, history, from_start, move_ids=None):
        """One position by its game history (records of _lib.BOARD_DTYPE, oldest first, the position itself last)
        instead of its planes: EncodePositionForNN (src/neural/encoder.cc:134) runs on the device."""
        h = np.ascontiguousarray(history, _lib.BOARD_DTYPE).reshape(-1)
        if move_ids is None:
            _lib.check(self._lib.b200_comp_add_position(self._h, h.ctypes.data, h.size, 1 if from_start else 0, None, -1))
        else:
            ids = np.ascontiguousarray(move_ids, np.uint16).reshape(-1)
            _lib.check(self._lib.b200_comp_add_position(self._h, h.ctypes.data, h.size, 1 if from_start else 0,
                                                        ids.ctypes.data, ids.size))

    def add_positions(self, boards, offsets, from_start, move_ids=None, n_moves=None):
        """Batch form of add_position: concatenated histories with n + 1 offsets; move_ids [n][256], n_moves [n]."""
        b = np.ascontiguousarray(boards, _lib.BOARD_DTYPE).reshape(-1)
        o = np.ascontiguousarray(offsets, np.int32).reshape(-1)
        f = np.ascontiguousarray(from_start, np.uint8).reshape(-1)
        n = f.size
        if o.size != n + 1:
            raise ValueError("offsets must have one entry more than from_start")
        if move_ids is None:
            _lib.check(self._lib.b200_comp_add_positions(self._h, b.ctypes.data, o.ctypes.data, f.ctypes.data, None, None, n))
        else:
            ids = np.ascontiguousarray(move_ids, np.uint16).reshape(n, 256)
            cnt = np.ascontiguousarray(n_moves, np.int32).reshape(n)
            _lib.check(self._lib.b200_comp_add_positions(self._h, b.ctypes.data, o.ctypes.data, f.ctypes.data,
                                                         ids.ctypes.data, cnt.ctypes.data, n))

    def set_policy_options(self, temperature=1.0, compact=False):
        """Policy softmax temperature (the wrapper multiplies by 1/temperature) and compact return."""
        _lib.check(self._lib.b200_comp_set_policy_options(self._h, 1.0 / float(temperature), 1 if compact else 0))

    def legal_policy(self, sample):
        """Probabilities of the sample's legal moves, in the order the moves were given."""
        p = ctypes.POINTER(ctypes.c_float)()
        n = ctypes.c_int()
        _lib.check(self._lib.b200_comp_legal_policy(self._h, sample, ctypes.byref(p), ctypes.byref(n)))
        return np.ctypeslib.as_array(p, shape=(n.value,)).copy() if n.value else np.zeros(0, np.float32)

    def add_inputs(self, masks, values):
        m = np.ascontiguousarray(masks, np.uint64).reshape(-1, 112)
        v = np.ascontiguousarray(values, np.float32).reshape(-1, 112)
        if m.shape != v.shape:
            raise ValueError("masks and values must describe the same number of positions")
        _lib.check(self._lib.b200_comp_add_inputs(self._h, m.ctypes.data, v.ctypes.data, m.shape[0]))

    def compute_blocking(self):
        _lib.check(self._lib.b200_comp_compute(self._h))

    def get_batch_size(self):
        return self._lib.b200_comp_batch_size(self._h)

    def _chk(self, sample):
        if not 0 <= sample < self.get_batch_size():
            raise IndexError("sample %d out of range" % sample)

    def get_q_val(self, sample):
        self._chk(sample)
        return self._lib.b200_comp_q(self._h, sample)

    def get_d_val(self, sample):
        self._chk(sample)
        return self._lib.b200_comp_d(self._h, sample)

    def get_m_val(self, sample):
        self._chk(sample)
        return self._lib.b200_comp_m(self._h, sample)

    def get_p_val(self, sample, move_id):
        self._chk(sample)
        if not 0 <= move_id < _lib.POLICY_SIZE:
            raise IndexError("move id %d out of range" % move_id)
        return self._lib.b200_comp_p(self._h, sample, move_id)

    def policy(self, sample):
        """All 1858 raw logits of one sample (a copy)."""
        self._chk(sample)
        p = self._lib.b200_comp_policy(self._h, sample)
        return np.ctypeslib.as_array(p, shape=(_lib.POLICY_SIZE,)).copy()

    def close(self):
        if self._h:
            self._lib.b200_comp_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Network:
    """lczero::Network over b200_net."""

    def __init__(self, net, options=None):
        opts = parse_options(options)
        lib = _lib.load()
        self._lib = lib
        self._handle = None
        prec = str(opts.get("precision", "fp16")).lower()
        if prec not in _lib.PRECISIONS:
            raise ValueError("Unknown precision '%s'" % prec)
        meta, tensors = _weights.flatten(net, policy_head=opts.get("policy_head", "vanilla"),
                                         value_head=opts.get("value_head", "winner"))
        b = ctypes.c_void_p()
        _lib.check(lib.b200_builder_create(ctypes.byref(b)))
        try:
            for k, v in meta.items():
                _lib.check(lib.b200_builder_set_int(b, k.encode(), int(v)))
            for name, arr in tensors.items():
                a = np.ascontiguousarray(arr, np.float32)
                _lib.check(lib.b200_builder_add_tensor(b, name.encode(), a.ctypes.data, a.size))
            o = _lib.NetOptions(gpu=int(opts.get("gpu", 0)), max_batch=int(opts.get("max_batch", 1024)),
                                precision=_lib.PRECISIONS[prec], slots=int(opts.get("slots", 1)),
                                mlh=1 if _as_bool(opts.get("mlh", True)) else 0,
                                flags=option_flags(opts))
            h = ctypes.c_void_p()
            _lib.check(lib.b200_net_create(b, ctypes.byref(o), ctypes.byref(h)))
            self._handle = h
        finally:
            lib.b200_builder_destroy(b)
        self.info = _lib.NetInfo()
        _lib.check(lib.b200_net_get_info(self._handle, ctypes.byref(self.info)))
        self.precision = prec

    # -- lczero::Network --
    def get_capabilities(self):
        return {"input_format": self.info.input_format, "output_format": self.info.output_format,
                "moves_left": self.info.moves_left_format if self.info.has_mlh else 0}

    def new_computation(self):
        return NetworkComputation(self)

    def get_threads(self):
        return 1

    def is_cpu(self):
        return False

    def get_mini_batch_size(self):
        return 2 * self.info.sm_count

    def get_preferred_batch_step(self):
        return 1

    # -- whole-batch helpers --
    def evaluate(self, masks, values):
        """Evaluate host arrays in one call; returns dict(policy, q, d, m)."""
        m = np.ascontiguousarray(masks, np.uint64).reshape(-1, 112)
        v = np.ascontiguousarray(values, np.float32).reshape(-1, 112)
        n = m.shape[0]
        out = dict(policy=np.empty((n, 1858), np.float32), q=np.empty(n, np.float32),
                   d=np.empty(n, np.float32), m=np.empty(n, np.float32))
        _lib.check(self._lib.b200_net_eval_host(self._handle, m.ctypes.data, v.ctypes.data, n,
                                                out["policy"].ctypes.data, out["q"].ctypes.data,
                                                out["d"].ctypes.data, out["m"].ctypes.data))
        return out

    def new_mux(self, max_batch=None, wait_us=200):
        """Batch aggregator over this network: see Mux."""
        return Mux(self, max_batch or self.info.max_batch, wait_us)

    def enqueue_device(self, d_masks, d_values, n, d_policy, d_qdm):
        _lib.check(self._lib.b200_net_enqueue_device(self._handle, d_masks, d_values, n, d_policy, d_qdm))

    def sync(self):
        _lib.check(self._lib.b200_net_sync(self._handle))

    def stream(self):
        return self._lib.b200_net_stream(self._handle)

    def launch_count(self):
        return self._lib.b200_net_launch_count(self._handle)

    def device_status(self):
        return self._lib.b200_net_device_status(self._handle)

    def inject_device_status(self, code):
        """Test hook: make the next evaluation of every slot fail the way a kernel that gave up would."""
        _lib.check(self._lib.b200_net_inject_device_status(self._handle, int(code)))

    PROFILE_CLASSES = ("gemm_tc", "gemm_fma", "attention", "layer_norm", "other")

    def set_profiling(self, enabled):
        _lib.check(self._lib.b200_net_set_profiling(self._handle, 1 if enabled else 0))

    def get_profile(self, reset=True):
        """{class: dict(ms, work, launches)}: device time, algorithmic FLOPs (GEMMs) or bytes."""
        k = len(self.PROFILE_CLASSES)
        ms, work, cnt = np.zeros(k), np.zeros(k), np.zeros(k, np.int64)
        _lib.check(self._lib.b200_net_get_profile(self._handle, ms.ctypes.data, work.ctypes.data,
                                                  cnt.ctypes.data, 1 if reset else 0))
        return {c: dict(ms=float(ms[i]), work=float(work[i]), launches=int(cnt[i]))
                for i, c in enumerate(self.PROFILE_CLASSES)}

    PROFILE_TAGS = ("untagged", "qkv", "out_proj", "ffn1", "ffn2", "smolgen_dense", "smolgen_bias", "attention",
                    "embedding", "heads")

    def get_profile_tagged(self, reset=True):
        """{tag: dict(ms, work, launches)} of the launches that carry a tag: which product of the encoder layer."""
        k = 16
        ms, work, cnt = np.zeros(k), np.zeros(k), np.zeros(k, np.int64)
        _lib.check(self._lib.b200_net_get_profile_tagged(self._handle, ms.ctypes.data, work.ctypes.data,
                                                         cnt.ctypes.data, 1 if reset else 0))
        return {c: dict(ms=float(ms[i]), work=float(work[i]), launches=int(cnt[i]))
                for i, c in enumerate(self.PROFILE_TAGS) if i > 0}

    def close(self):
        if self._handle:
            self._lib.b200_net_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def create_network(weights_path_or_net, options=None):
    """Factory: a weights file path (or parsed Net dict) plus options -> Network."""
    if weights_path_or_net is None:
        raise ValueError("The b200 backend requires a network file.")
    net = weights_path_or_net
    if not isinstance(net, dict):
        net = netproto.load_net(net)
    return Network(net, options)


class Mux:
    """Many caller threads, one GPU batch: blocking `evaluate` calls from different threads are merged (the role of
    lc0's `multiplexing` backend, src/neural/backends/network_mux.cc:169-205)."""

    def __init__(self, network, max_batch, wait_us):
        self._lib = _lib.load()
        self._network = network  # keeps the network alive
        h = ctypes.c_void_p()
        _lib.check(self._lib.b200_mux_create(network._handle, int(max_batch), int(wait_us), ctypes.byref(h)))
        self._h = h

    def evaluate(self, masks, values):
        m = np.ascontiguousarray(masks, np.uint64).reshape(-1, 112)
        v = np.ascontiguousarray(values, np.float32).reshape(-1, 112)
        n = m.shape[0]
        out = dict(policy=np.empty((n, 1858), np.float32), q=np.empty(n, np.float32),
                   d=np.empty(n, np.float32), m=np.empty(n, np.float32))
        _lib.check(self._lib.b200_mux_eval(self._h, m.ctypes.data, v.ctypes.data, n, out["policy"].ctypes.data,
                                           out["q"].ctypes.data, out["d"].ctypes.data, out["m"].ctypes.data))
        return out

    def stats(self):
        r, b, p = ctypes.c_longlong(), ctypes.c_longlong(), ctypes.c_longlong()
        _lib.check(self._lib.b200_mux_stats(self._h, ctypes.byref(r), ctypes.byref(b), ctypes.byref(p)))
        return dict(requests=r.value, batches=b.value, positions=p.value)

    def close(self):
        if self._h:
            self._lib.b200_mux_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass


class MultiGpuNetwork:
    """One batch over several GPUs of the box: contiguous slices, replicated weights, no exchange (the role of lc0's
    `demux` backend, src/neural/backends/network_demux.cc:279-334).  `options` as for Network plus
    `gpus=0+1+2` (or a list); `max_batch` is per GPU."""

    def __init__(self, net, options=None, gpus=None):
        opts = parse_options(options)
        lib = _lib.load()
        self._lib = lib
        self._h = None
        if gpus is None:
            gpus = [int(g) for g in str(opts.get("gpus", "0")).replace("+", " ").split()]
        prec = str(opts.get("precision", "fp16")).lower()
        if prec not in _lib.PRECISIONS:
            raise ValueError("Unknown precision '%s'" % prec)
        meta, tensors = _weights.flatten(net, policy_head=opts.get("policy_head", "vanilla"),
                                         value_head=opts.get("value_head", "winner"))
        b = ctypes.c_void_p()
        _lib.check(lib.b200_builder_create(ctypes.byref(b)))
        try:
            for k, v in meta.items():
                _lib.check(lib.b200_builder_set_int(b, k.encode(), int(v)))
            for name, arr in tensors.items():
                a = np.ascontiguousarray(arr, np.float32)
                _lib.check(lib.b200_builder_add_tensor(b, name.encode(), a.ctypes.data, a.size))
            o = _lib.NetOptions(gpu=0, max_batch=int(opts.get("max_batch", 1024)), precision=_lib.PRECISIONS[prec],
                                slots=int(opts.get("slots", 1)), mlh=1 if _as_bool(opts.get("mlh", True)) else 0,
                                flags=option_flags(opts))
            ids = (ctypes.c_int * len(gpus))(*gpus)
            h = ctypes.c_void_p()
            _lib.check(lib.b200_multi_create(b, ctypes.byref(o), ids, len(gpus), ctypes.byref(h)))
            self._h = h
        finally:
            lib.b200_builder_destroy(b)
        self.gpus = list(gpus)

    def evaluate(self, masks, values):
        m = np.ascontiguousarray(masks, np.uint64).reshape(-1, 112)
        v = np.ascontiguousarray(values, np.float32).reshape(-1, 112)
        n = m.shape[0]
        out = dict(policy=np.empty((n, 1858), np.float32), q=np.empty(n, np.float32),
                   d=np.empty(n, np.float32), m=np.empty(n, np.float32))
        _lib.check(self._lib.b200_multi_eval_host(self._h, m.ctypes.data, v.ctypes.data, n, out["policy"].ctypes.data,
                                                  out["q"].ctypes.data, out["d"].ctypes.data, out["m"].ctypes.data))
        return out

    def close(self):
        if self._h:
            self._lib.b200_multi_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass
