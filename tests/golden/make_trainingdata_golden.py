"""Generate tests/golden/trainingdata_golden.npz (run where the reference is built: python oracle/build_ref.py).

The fields of V6 training-data records that the plane reader uses, written for seeded game histories the way the
reference's writer fills them, the planes the reference's own PlanesFromTrainingData (src/trainingdata/reader.cc:32-118)
reads back, and the planes EncodePositionForNN produced for the same position (oracle/_ref/mktd).

usage: python tests/golden/make_trainingdata_golden.py [count]
"""
import os
import struct
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))

REC = np.dtype([("input_format", "<u4"), ("planes", "<u8", (104,)), ("bytes", "u1", (8,)),
                ("reader_masks", "<u8", (112,)), ("reader_values", "<f4", (112,)),
                ("encoder_masks", "<u8", (112,)), ("encoder_values", "<f4", (112,))])


def main():
    count = int(sys.argv[1]) if len(sys.argv) > 1 else 160
    exe = os.path.join(ROOT, "oracle", "_ref", "mktd")
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "td.bin")
        subprocess.run([exe, path, str(count)], check=True)
        raw = open(path, "rb").read()
    assert raw[:8] == b"LC0TDV6\0"
    n = struct.unpack_from("<i", raw, 8)[0]
    recs = np.frombuffer(raw, REC, n, 12)
    assert 12 + n * REC.itemsize == len(raw)
    np.savez_compressed(os.path.join(HERE, "trainingdata_golden.npz"), input_format=recs["input_format"],
                        planes=recs["planes"], bytes=recs["bytes"][:, :7], reader_masks=recs["reader_masks"],
                        reader_values=recs["reader_values"], encoder_masks=recs["encoder_masks"],
                        encoder_values=recs["encoder_values"])
    inv = recs["bytes"][:, 6] & 7
    print("records", n, "transform histogram", np.bincount(inv, minlength=8))


if __name__ == "__main__":
    main()
