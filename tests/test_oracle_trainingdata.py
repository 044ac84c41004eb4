"""The training-data plane reader restatement (oracle/encoder.py planes_from_training_data) against the reference's
PlanesFromTrainingData and EncodePositionForNN outputs (tests/golden/trainingdata_golden.npz): bit-exact."""
import os

import numpy as np

from conftest import ROOT
from oracle import encoder

GOLDEN = os.path.join(ROOT, "tests", "golden", "trainingdata_golden.npz")


def test_reader_restatement_is_bit_exact_against_the_reference():
    g = np.load(GOLDEN)
    n = len(g["input_format"])
    assert n >= 500
    transforms = set()
    for i in range(n):
        fmt = int(g["input_format"][i])
        m, v = encoder.planes_from_training_data(fmt, g["planes"][i], g["bytes"][i], True)
        assert np.array_equal(m, g["reader_masks"][i]), (i, fmt)
        assert np.array_equal(v.view(np.uint32), g["reader_values"][i].view(np.uint32)), (i, fmt)
        # without taking the transform back the record reads as the planes the encoder produced for the position
        m, v = encoder.planes_from_training_data(fmt, g["planes"][i], g["bytes"][i], False)
        assert np.array_equal(m, g["encoder_masks"][i]), (i, fmt)
        assert np.array_equal(v.view(np.uint32), g["encoder_values"][i].view(np.uint32)), (i, fmt)
        transforms.add(int(g["bytes"][i][6]) & 7)
    assert transforms == set(range(8))


def test_record_offsets_match_the_packed_struct():
    assert encoder.TD_OFF_PLANES == 7440 and encoder.TD_OFF_BYTES == 8272 and encoder.TD_RECORD_BYTES == 8356
