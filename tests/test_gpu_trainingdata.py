"""Device-side reader of V6 training-data records against the reference's PlanesFromTrainingData and
EncodePositionForNN outputs (bit-exact), and the records evaluated by a network."""
import os

import numpy as np
import pytest
import torch

from conftest import ROOT, load_case
from lc0_b200 import _lib, network
from oracle import encoder

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(ROOT, "tests", "golden", "trainingdata_golden.npz")


def _records(g, stride=encoder.TD_RECORD_BYTES):
    """Full-size packed records with the fixture's fields in place and everything else zero."""
    n = len(g["input_format"])
    raw = np.zeros((n, stride), np.uint8)
    raw[:, 0:4] = np.frombuffer(np.full(n, 6, "<u4").tobytes(), np.uint8).reshape(n, 4)
    raw[:, 4:8] = np.frombuffer(g["input_format"].astype("<u4").tobytes(), np.uint8).reshape(n, 4)
    raw[:, encoder.TD_OFF_PLANES:encoder.TD_OFF_BYTES] = np.frombuffer(
        np.ascontiguousarray(g["planes"], "<u8").tobytes(), np.uint8).reshape(n, 832)
    raw[:, encoder.TD_OFF_BYTES:encoder.TD_OFF_BYTES + 7] = g["bytes"]
    return raw


@pytest.mark.parametrize("stride", [8356, 8396])  # V6 records, and a longer record type with the same prefix
def test_reader_kernel_is_bit_exact(stride):
    lib = _lib.load()
    g = np.load(GOLDEN)
    n = len(g["input_format"])
    rec = torch.from_numpy(_records(g, stride)).cuda()
    for undo, mk, vk in ((1, "reader_masks", "reader_values"), (0, "encoder_masks", "encoder_values")):
        masks = torch.zeros(n, 112, dtype=torch.int64, device="cuda")
        values = torch.zeros(n, 112, dtype=torch.float32, device="cuda")
        bad = torch.zeros(1, dtype=torch.int32, device="cuda")
        _lib.check(lib.b200_op_planes_from_training_data(rec.data_ptr(), n, stride, undo, masks.data_ptr(),
                                                         values.data_ptr(), bad.data_ptr(), None))
        torch.cuda.synchronize()
        assert int(bad.item()) == 0
        assert np.array_equal(masks.cpu().numpy().view(np.uint64), g[mk])
        assert np.array_equal(values.cpu().numpy().view(np.uint32), g[vk].view(np.uint32))


def test_unknown_format_is_counted_and_bad_arguments_rejected():
    lib = _lib.load()
    g = np.load(GOLDEN)
    raw = _records(g)[:8].copy()
    raw[3, 4:8] = np.frombuffer(np.array([7], "<u4").tobytes(), np.uint8)
    rec = torch.from_numpy(raw).cuda()
    masks = torch.ones(8, 112, dtype=torch.int64, device="cuda")
    values = torch.zeros(8, 112, dtype=torch.float32, device="cuda")
    bad = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.check(lib.b200_op_planes_from_training_data(rec.data_ptr(), 8, 8356, 0, masks.data_ptr(), values.data_ptr(),
                                                     bad.data_ptr(), None))
    torch.cuda.synchronize()
    assert int(bad.item()) == 1 and not masks[3].any()
    assert lib.b200_op_planes_from_training_data(rec.data_ptr(), 8, 100, 0, masks.data_ptr(), values.data_ptr(), None,
                                                 None) == _lib.ERR_INVALID
    assert lib.b200_op_planes_from_training_data(None, 0, 8356, 0, None, None, None, None) == _lib.OK


def test_records_feed_a_network_like_the_encoded_positions():
    """Records -> planes on the device -> b200_net_eval_device gives what the encoder's planes give."""
    lib = _lib.load()
    g = np.load(GOLDEN)
    sel = np.nonzero(g["input_format"] == 2)[0][:32]
    net, pos, n, gold = load_case("cfg3_mini")  # input format 2
    nw = network.Network(net, "precision=fp32,max_batch=32")
    want = nw.evaluate(g["encoder_masks"][sel], g["encoder_values"][sel])
    sub = {k: g[k][sel] for k in ("input_format", "planes", "bytes")}
    rec = torch.from_numpy(_records(sub)).cuda()
    masks = torch.zeros(len(sel), 112, dtype=torch.int64, device="cuda")
    values = torch.zeros(len(sel), 112, dtype=torch.float32, device="cuda")
    _lib.check(lib.b200_op_planes_from_training_data(rec.data_ptr(), len(sel), 8356, 0, masks.data_ptr(),
                                                     values.data_ptr(), None, None))
    torch.cuda.synchronize()
    policy = torch.zeros(len(sel), 1858, device="cuda")
    qdm = torch.zeros(len(sel), 3, device="cuda")
    nw.enqueue_device(masks.data_ptr(), values.data_ptr(), len(sel), policy.data_ptr(), qdm.data_ptr())
    nw.sync()
    assert np.array_equal(policy.cpu().numpy(), want["policy"])
    assert np.array_equal(qdm.cpu().numpy()[:, 0], want["q"])
    nw.close()
