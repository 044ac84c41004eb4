"""ctypes binding of libb200nn.so (the C ABI declared in include/b200nn.h).

There is no fallback: if the shared object is missing or a symbol cannot be
resolved, importing fails loudly; if no CUDA device is usable, network creation fails.
"""
import ctypes

import numpy as np
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200nn.so")

OK, ERR_INVALID, ERR_CUDA, ERR_UNSUPPORTED, ERR_NOMEM, ERR_TIMEOUT = range(6)
PREC_FP32, PREC_FP16, PREC_BF16 = 0, 1, 2
PRECISIONS = {"fp32": PREC_FP32, "fp16": PREC_FP16, "bf16": PREC_BF16}
FLAG_NO_TENSOR_CORES = 1
FLAG_NO_GRAPHS = 2
FLAG_NO_LN_FOLD = 4
FLAG_NO_MERGED_COMPRESS = 8
FLAG_NO_SPLIT_LAST_WAVE = 16
FLAG_NO_FUSED_SE = 32
FLAG_WINOGRAD = 64
FLAG_NO_SIDE_STREAM = 128
FLAG_NO_DEPENDENT_LAUNCH = 256
FLAG_NO_TOWER_KERNEL = 512
POLICY_SIZE = 1858
INPUT_PLANES = 112


class B200Error(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("b200nn error %d: %s" % (code, msg))
        self.code = code


class NetOptions(ctypes.Structure):
    _fields_ = [("gpu", ctypes.c_int), ("max_batch", ctypes.c_int), ("precision", ctypes.c_int),
                ("slots", ctypes.c_int), ("mlh", ctypes.c_int), ("flags", ctypes.c_int)]


class GemmDesc(ctypes.Structure):
    """b200_gemm_desc (include/b200nn.h)."""
    _fields_ = [("A", ctypes.c_void_p), ("W", ctypes.c_void_p), ("bias", ctypes.c_void_p), ("C", ctypes.c_void_p),
                ("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int),
                ("lda", ctypes.c_longlong), ("ldw", ctypes.c_longlong), ("ldc", ctypes.c_longlong),
                ("activation", ctypes.c_int), ("precision", ctypes.c_int),
                ("scale", ctypes.c_float), ("alpha", ctypes.c_float),
                ("a_stats", ctypes.c_void_p), ("colsum", ctypes.c_void_p),
                ("a_inv_c", ctypes.c_float), ("a_eps", ctypes.c_float),
                ("res", ctypes.c_void_p), ("ldres", ctypes.c_longlong),
                ("res_stats", ctypes.c_void_p), ("res_gamma", ctypes.c_void_p), ("res_beta", ctypes.c_void_p),
                ("res_inv_c", ctypes.c_float), ("res_eps", ctypes.c_float),
                ("out_stats", ctypes.c_void_p),
                ("C2", ctypes.c_void_p), ("ldc2", ctypes.c_longlong), ("n_split", ctypes.c_int),
                ("whole_tiles", ctypes.c_int)]


class NetInfo(ctypes.Structure):
    _fields_ = [("input_format", ctypes.c_int), ("output_format", ctypes.c_int),
                ("moves_left_format", ctypes.c_int), ("wdl", ctypes.c_int), ("has_mlh", ctypes.c_int),
                ("attention_body", ctypes.c_int), ("embedding", ctypes.c_int),
                ("encoder_layers", ctypes.c_int), ("heads", ctypes.c_int), ("dff", ctypes.c_int),
                ("filters", ctypes.c_int), ("residual_blocks", ctypes.c_int), ("max_batch", ctypes.c_int),
                ("precision", ctypes.c_int), ("sm_count", ctypes.c_int),
                ("weight_bytes", ctypes.c_longlong), ("workspace_bytes", ctypes.c_longlong),
                ("flops_per_position", ctypes.c_double), ("gemm_flops_per_position", ctypes.c_double)]


_P = ctypes.c_void_p
_I = ctypes.c_int
_F = ctypes.c_float
# name -> (restype, argtypes); every symbol include/b200nn.h declares.
SIGNATURES = {
    "b200_last_error": (ctypes.c_char_p, []),
    "b200_builder_create": (_I, [ctypes.POINTER(_P)]),
    "b200_builder_set_int": (_I, [_P, ctypes.c_char_p, ctypes.c_longlong]),
    "b200_builder_add_tensor": (_I, [_P, ctypes.c_char_p, _P, ctypes.c_size_t]),
    "b200_builder_destroy": (None, [_P]),
    "b200_net_create": (_I, [_P, ctypes.POINTER(NetOptions), ctypes.POINTER(_P)]),
    "b200_net_get_info": (_I, [_P, ctypes.POINTER(NetInfo)]),
    "b200_net_destroy": (None, [_P]),
    "b200_comp_create": (_I, [_P, ctypes.POINTER(_P)]),
    "b200_comp_add_input": (_I, [_P, _P, _P]),
    "b200_comp_add_inputs": (_I, [_P, _P, _P, _I]),
    "b200_comp_compute": (_I, [_P]),
    "b200_comp_batch_size": (_I, [_P]),
    "b200_comp_q": (_F, [_P, _I]),
    "b200_comp_d": (_F, [_P, _I]),
    "b200_comp_m": (_F, [_P, _I]),
    "b200_comp_p": (_F, [_P, _I, _I]),
    "b200_comp_policy": (ctypes.POINTER(_F), [_P, _I]),
    "b200_comp_destroy": (None, [_P]),
    "b200_comp_add_input_with_moves": (_I, [_P, _P, _P, _P, _I]),
    "b200_comp_add_inputs_with_moves": (_I, [_P, _P, _P, _P, _P, _I]),
    "b200_comp_set_policy_options": (_I, [_P, _F, _I]),
    "b200_comp_legal_policy": (_I, [_P, _I, ctypes.POINTER(ctypes.POINTER(_F)), ctypes.POINTER(_I)]),
    "b200_comp_set_encoding": (_I, [_P, _I, _I]),
    "b200_comp_add_position": (_I, [_P, _P, _I, _I, _P, _I]),
    "b200_comp_add_positions": (_I, [_P, _P, _P, _P, _P, _P, _I]),
    "b200_mux_create": (_I, [_P, _I, _I, ctypes.POINTER(_P)]),
    "b200_mux_eval": (_I, [_P, _P, _P, _I, _P, _P, _P, _P]),
    "b200_mux_stats": (_I, [_P, ctypes.POINTER(ctypes.c_longlong), ctypes.POINTER(ctypes.c_longlong),
                            ctypes.POINTER(ctypes.c_longlong)]),
    "b200_mux_destroy": (None, [_P]),
    "b200_multi_slice": (None, [_I, _I, _I, ctypes.POINTER(_I), ctypes.POINTER(_I)]),
    "b200_multi_create": (_I, [_P, _P, ctypes.POINTER(_I), _I, ctypes.POINTER(_P)]),
    "b200_multi_gpu_count": (_I, [_P]),
    "b200_multi_net": (_P, [_P, _I]),
    "b200_multi_eval_host": (_I, [_P, _P, _P, _I, _P, _P, _P, _P]),
    "b200_multi_destroy": (None, [_P]),
    "b200_net_eval_host": (_I, [_P, _P, _P, _I, _P, _P, _P, _P]),
    "b200_net_eval_device": (_I, [_P, _P, _P, _I, _P, _P]),
    "b200_net_enqueue_device": (_I, [_P, _P, _P, _I, _P, _P]),
    "b200_net_sync": (_I, [_P]),
    "b200_net_stream": (_P, [_P]),
    "b200_net_launch_count": (ctypes.c_longlong, [_P]),
    "b200_net_device_status": (_I, [_P]),
    "b200_net_inject_device_status": (_I, [_P, _I]),
    "b200_net_get_profile_tagged": (_I, [_P, _P, _P, _P, _I]),
    "b200_net_set_profiling": (_I, [_P, _I]),
    "b200_net_get_profile": (_I, [_P, _P, _P, _P, _I]),
    "b200_op_expand_planes": (_I, [_P, _P, _I, _P, _I, _P]),
    "b200_op_encode_positions": (_I, [_P, _P, _P, _I, _I, _I, _P, _P, _P, _P]),
    "b200_op_planes_from_training_data": (_I, [_P, _I, ctypes.c_longlong, _I, _P, _P, _P, _P]),
    "b200_op_gemm": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P]),
    "b200_op_scratch_residency_probe": (_I, [_I, _I, _I, _I, ctypes.POINTER(ctypes.c_float)]),
    "b200_op_gemm_ex": (_I, [ctypes.POINTER(GemmDesc), _P]),
    "b200_op_attention": (_I, [_P, _P, _P, ctypes.c_longlong, _P, _P, ctypes.c_longlong, _I, _I, _I, _I, _I, _P]),
    "b200_op_gemm_timed": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, ctypes.POINTER(ctypes.c_float), _P]),
    "b200_op_policy_attention": (_I, [_P, _P, _P, _I, _I, _P, _P, _I, _P]),
    "b200_op_policy_attention_static": (_I, [_P, _P, _P, _I, _I, _P, _I, _P]),
    "b200_op_layer_norm": (_I, [_P, _P, _P, _P, _P, _I, _I, _F, _F, _I, _P]),
}

# struct b200_board (include/b200nn.h), 88 bytes
BOARD_DTYPE = np.dtype([
    ("ours", "<u8"), ("theirs", "<u8"), ("pawns", "<u8"), ("knights", "<u8"), ("bishops", "<u8"), ("rooks", "<u8"),
    ("queens", "<u8"), ("kings", "<u8"), ("en_passant", "<u8"), ("castling", "u1"), ("rook_files", "u1", (4,)),
    ("flags", "u1"), ("rule50", "<u2"), ("repetitions", "u1"), ("reserved", "u1", (7,))])
FILL_NO, FILL_FEN_ONLY, FILL_ALWAYS = 0, 1, 2

_lib = None


def load():
    """Load the shared object (once) and bind every declared symbol."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError("%s is missing: build it with `python -m lc0_b200.build` "
                          "(there is no CPU fallback)" % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(code):
    if code != OK:
        raise B200Error(code, load().b200_last_error().decode("utf-8", "replace"))
