"""Policy / positional-encoding tables generated from chess geometry."""
import os
import re

import numpy as np
import pytest

from oracle import tables

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(os.environ.get("LC0_REFERENCE", os.path.join(os.path.dirname(_ROOT), "reference")), "src", "neural")


def test_table_shapes_and_bijection():
    assert len(tables.move_strings()) == 1858
    am = tables.attn_policy_map()
    cm = tables.conv_policy_map()
    assert am.shape == (64 * 64 + 8 * 24,) and cm.shape == (73 * 64,)
    # every policy index is produced exactly once by each head layout
    assert sorted(am[am >= 0].tolist()) == list(range(1858))
    assert sorted(cm[cm >= 0].tolist()) == list(range(1858))
    pe = tables.pos_encoding()
    assert pe.shape == (64, 64) and np.all(np.diag(pe) == -1)
    assert pe[0, 1] == 1 and pe[0, 10] == 1 and pe[0, 11] == 0  # a1-b1 rook, a1-c2 knight, a1-d2 nothing


def _ints(text, start_token):
    a = text.index(start_token)
    b = text.index("};", a)
    return np.array([int(x) for x in re.findall(r"-?\d+", text[a + len(start_token):b])])


@pytest.mark.skipif(not os.path.isdir(REF), reason="reference tree not present")
def test_tables_equal_reference_arrays():
    enc = open(os.path.join(REF, "encoder.cc")).read()
    a = enc.index("kMoveStrs[] = {")
    mv = re.findall(r'"([a-h][1-8][a-h][1-8][qrbn]?)"', enc[a:enc.index("};", a)])
    assert tuple(mv) == tables.move_strings()
    pm = open(os.path.join(REF, "tables", "policy_map.h")).read()
    assert np.array_equal(_ints(pm, "kConvPolicyMap[] = {"), tables.conv_policy_map())
    ap = open(os.path.join(REF, "tables", "attention_policy_map.h")).read()
    assert np.array_equal(_ints(ap, "kAttnPolicyMap[] = {"), tables.attn_policy_map())
    a = ap.index("kPosEncoding[64][kNumPosEncodingChannels] = {")
    pe = np.array([float(x) for x in re.findall(r"-?\d+\.\d+", ap[a + 45:ap.index("};", a)])])
    assert np.array_equal(pe.reshape(64, 64), tables.pos_encoding())
