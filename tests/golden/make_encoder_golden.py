"""Generate tests/golden/encoder_golden.npz (run where the reference is built: python oracle/build_ref.py).

Seeded game histories (random legal playouts from the standard position and from a few others that reach every board
transform, en-passant starts and Chess960 rook files) as `b200_board` records, and the planes the reference's own
EncodePositionForNN (src/neural/encoder.cc:134-328) produces for them under every input format and fill policy
(oracle/_ref/mkenc).  Pins oracle/encoder.py and the device-side encoder bit-exactly.

usage: python tests/golden/make_encoder_golden.py [count]
"""
import os
import struct
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import encoder  # noqa: E402


def read_enc(path):
    raw = open(path, "rb").read()
    assert raw[:8] == b"LC0ENC1\0"
    n, n_combos = struct.unpack_from("<ii", raw, 8)
    off = 16
    combos = np.frombuffer(raw, "<i4", n_combos * 2, off).reshape(n_combos, 2).copy()
    off += n_combos * 8
    boards, offsets, from_start = [], [0], []
    masks = np.zeros((n, n_combos, 112), np.uint64)
    values = np.zeros((n, n_combos, 112), np.float32)
    transforms = np.zeros((n, n_combos), np.int32)
    for s in range(n):
        cnt, fs = struct.unpack_from("<ii", raw, off)
        off += 8
        boards.append(np.frombuffer(raw, encoder.BOARD_DTYPE, cnt, off).copy())
        off += cnt * encoder.BOARD_DTYPE.itemsize
        offsets.append(offsets[-1] + cnt)
        from_start.append(fs)
        for c in range(n_combos):
            masks[s, c] = np.frombuffer(raw, "<u8", 112, off)
            off += 112 * 8
            values[s, c] = np.frombuffer(raw, "<f4", 112, off)
            off += 112 * 4
            transforms[s, c] = struct.unpack_from("<i", raw, off)[0]
            off += 4
    assert off == len(raw)
    return dict(boards=np.concatenate(boards), offsets=np.array(offsets, np.int32),
                from_start=np.array(from_start, np.uint8), combos=combos, masks=masks, values=values,
                transforms=transforms)


def main():
    count = int(sys.argv[1]) if len(sys.argv) > 1 else 192
    exe = os.path.join(ROOT, "oracle", "_ref", "mkenc")
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "enc.bin")
        subprocess.run([exe, path, str(count)], check=True)
        d = read_enc(path)
    np.savez_compressed(os.path.join(HERE, "encoder_golden.npz"), **d)
    t = d["transforms"]
    print("samples", count, "boards", len(d["boards"]), "transform histogram", np.bincount(t[t >= 0], minlength=8),
          "skipped combos", int((t < 0).sum()))


if __name__ == "__main__":
    main()
