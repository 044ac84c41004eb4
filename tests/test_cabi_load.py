"""The C-ABI library loads and exports every symbol include/b200nn.h declares (no compute)."""
import ctypes
import os
import re

import pytest

from conftest import ROOT
from lc0_b200 import _lib, mknet, network


def test_every_declared_symbol_is_exported(lib):
    header = open(os.path.join(ROOT, "include", "b200nn.h")).read()
    declared = set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", header))
    assert declared == set(_lib.SIGNATURES)
    for name in declared:
        assert hasattr(lib, name), name


def test_builder_argument_checks(lib):
    b = ctypes.c_void_p()
    assert lib.b200_builder_create(ctypes.byref(b)) == _lib.OK
    assert lib.b200_builder_set_int(b, b"network", 6) == _lib.OK
    assert lib.b200_builder_add_tensor(b, b"x", None, 4) == _lib.ERR_INVALID
    assert b"null" in lib.b200_last_error()
    lib.b200_builder_destroy(b)
    assert lib.b200_net_create(None, None, None) == _lib.ERR_INVALID


def test_option_parsing():
    assert network.parse_options("gpu=1, max_batch=512") == {"gpu": "1", "max_batch": "512"}
    with pytest.raises(ValueError, match="Unknown backend option"):
        network.parse_options("gpus=1")
    with pytest.raises(ValueError):
        network.parse_options("gpu")
    with pytest.raises(ValueError, match="requires a network file"):
        network.create_network(None)


def test_no_silent_cpu_fallback():
    """Without a CUDA device the product path must fail loudly instead of computing on the host."""
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        pytest.skip("a GPU is present")
    with pytest.raises(_lib.B200Error, match="CUDA"):
        network.Network(mknet.make_net("cfg3_mini"), "precision=fp32")
