"""Device-side position encoder against the reference's own EncodePositionForNN outputs (bit-exact) and, at the
computation level, against the same positions added as planes."""
import os

import numpy as np
import pytest
import torch

from conftest import ROOT, load_case
from lc0_b200 import _lib, network
from oracle import encoder

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(ROOT, "tests", "golden", "encoder_golden.npz")


@pytest.fixture(scope="module")
def lib():
    return _lib.load()


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def _encode_on_device(lib, g, fmt, fill):
    boards = torch.from_numpy(g["boards"].view(np.uint8).reshape(-1, 88).copy()).cuda()
    offsets = torch.from_numpy(g["offsets"].astype(np.int32)).cuda()
    from_start = torch.from_numpy(g["from_start"].astype(np.uint8)).cuda()
    n = len(g["from_start"])
    masks = torch.zeros(n, 112, dtype=torch.int64, device="cuda")
    values = torch.zeros(n, 112, dtype=torch.float32, device="cuda")
    transforms = torch.full((n,), -7, dtype=torch.int32, device="cuda")
    _lib.check(lib.b200_op_encode_positions(boards.data_ptr(), offsets.data_ptr(), from_start.data_ptr(), n, fmt, fill,
                                            masks.data_ptr(), values.data_ptr(), transforms.data_ptr(), None))
    torch.cuda.synchronize()
    return masks.cpu().numpy().view(np.uint64), values.cpu().numpy(), transforms.cpu().numpy()


def test_encoder_kernel_is_bit_exact_for_every_format_and_fill(lib, golden):
    checked = 0
    for c, (fmt, fill) in enumerate(golden["combos"]):
        m, v, t = _encode_on_device(lib, golden, int(fmt), int(fill))
        ok = golden["transforms"][:, c] >= 0  # combinations the reference does not terminate on are left out
        assert np.array_equal(t[ok], golden["transforms"][ok, c]), (fmt, fill)
        assert np.array_equal(m[ok], golden["masks"][ok, c]), (fmt, fill)
        assert np.array_equal(v[ok].view(np.uint32), golden["values"][ok, c].view(np.uint32)), (fmt, fill)
        checked += int(ok.sum())
    assert checked > 3000


def test_encoder_kernel_terminates_where_the_reference_does_not(lib, golden):
    """V2 format, history that starts at a position with a non-zero rule-50 counter, fill policy that walks past it:
    the kernel stops at the start of the history and agrees with the restatement."""
    c = [i for i, (f, fl) in enumerate(golden["combos"]) if f == 5 and fl == 2][0]
    skipped = np.nonzero(golden["transforms"][:, c] < 0)[0]
    assert len(skipped) > 0
    m, v, t = _encode_on_device(lib, golden, 5, 2)
    for s in skipped[:8]:
        hist = [encoder.board_from_record(r) for r in golden["boards"][golden["offsets"][s]:golden["offsets"][s + 1]]]
        wm, wv, wt = encoder.encode_position(hist, bool(golden["from_start"][s]), 5, 2)
        assert wt == t[s] and np.array_equal(wm, m[s]) and np.array_equal(wv, v[s])


def test_encoder_rejects_unknown_format_and_accepts_empty_batch(lib):
    assert lib.b200_op_encode_positions(None, None, None, 0, 1, 0, None, None, None, None) == _lib.OK
    d = torch.zeros(128, dtype=torch.uint8, device="cuda")
    rc = lib.b200_op_encode_positions(d.data_ptr(), d.data_ptr(), d.data_ptr(), 1, 7, 0, d.data_ptr(), d.data_ptr(), None,
                                      None)
    assert rc == _lib.ERR_UNSUPPORTED and b"Unsupported input plane encoding 7" in lib.b200_last_error()


def test_positions_added_by_history_evaluate_like_their_planes(golden):
    """Computation API: add_position (planes produced on the device) gives the same outputs as add_input with the
    reference-encoded planes, with and without the legal-move policy."""
    net, pos, n, g = load_case("cfg3_mini")  # input format 2
    nw = network.Network(net, "precision=fp32,max_batch=64")
    c_fmt = [i for i, (f, fl) in enumerate(golden["combos"]) if f == nw.info.input_format and fl == _lib.FILL_FEN_ONLY][0]
    count = 40
    offsets = golden["offsets"]
    a = nw.new_computation()
    a.add_inputs(golden["masks"][:count, c_fmt], golden["values"][:count, c_fmt])
    a.compute_blocking()
    b = nw.new_computation()
    for s in range(count):
        b.add_position(golden["boards"][offsets[s]:offsets[s + 1]], bool(golden["from_start"][s]))
    assert b.get_batch_size() == count
    b.compute_blocking()
    for s in range(count):
        assert np.array_equal(a.policy(s), b.policy(s))
        assert a.get_q_val(s) == b.get_q_val(s) and a.get_m_val(s) == b.get_m_val(s)
    # same with move lists, a different fill policy and the compact return; repeated so that the graph is replayed
    c_no = [i for i, (f, fl) in enumerate(golden["combos"]) if f == nw.info.input_format and fl == _lib.FILL_NO][0]
    moves = [np.arange(3 + s % 20, dtype=np.uint16) * 7 for s in range(count)]
    for rep in range(3):
        p = nw.new_computation()
        p.set_policy_options(1.0, compact=True)
        q = nw.new_computation()
        q.set_policy_options(1.0, compact=True)
        q.set_encoding(0, _lib.FILL_NO)
        for s in range(count):
            p.add_input_with_moves(golden["masks"][s, c_no], golden["values"][s, c_no], moves[s])
            q.add_position(golden["boards"][offsets[s]:offsets[s + 1]], bool(golden["from_start"][s]), moves[s])
        p.compute_blocking()
        q.compute_blocking()
        for s in range(count):
            assert np.array_equal(p.legal_policy(s), q.legal_policy(s))
        p.close()
        q.close()
    # batch form
    r = nw.new_computation()
    r.add_positions(golden["boards"][:offsets[count]], offsets[:count + 1], golden["from_start"][:count])
    r.compute_blocking()
    for s in range(count):
        assert np.array_equal(a.policy(s), r.policy(s))
    r.close()
    # mixing the two ways of adding inputs is an error
    with pytest.raises(_lib.B200Error):
        b.add_inputs(golden["masks"][:1, c_fmt], golden["values"][:1, c_fmt])
    a.close()
    b.close()
    assert nw.device_status() == 0
    nw.close()
