"""Generate the committed fixtures under tests/golden/ (run where the reference is built).

1. positions_*.npz  seeded random legal playouts encoded by the reference's own
   position encoder (oracle/_ref/mkpos): packed planes + legal-move policy indices.
2. golden_<net>.npz outputs of the reference's `blas` backend (oracle/_ref/ref_eval)
   for the seeded synthetic network <net> on the first positions of the matching
   position set, plus the legal-move softmax the reference's wrapper applies to them (computed by ref_eval with the
   reference's own FastExp).  These pin the numpy oracle; the reference has no vectors of its own.

usage: python tests/golden/make_golden.py   (after python oracle/build_ref.py)
"""
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from lc0_b200 import mknet  # noqa: E402

REF = os.path.join(ROOT, "oracle", "_ref")

POSITION_SETS = {  # name -> (count, input_format, mix)
    "positions_fmt1_uniform": (512, 1, "uniform"),
    "positions_fmt2_uniform": (1024, 2, "uniform"),
    "positions_fmt2_split": (1024, 2, "split"),
}
GOLDENS = {  # net -> (position set, count)
    "cfg1_mini": ("positions_fmt1_uniform", 32),
    "cfg2_mini": ("positions_fmt1_uniform", 32),
    "cfg3_mini": ("positions_fmt2_uniform", 32),
    "cfg4_mini": ("positions_fmt2_uniform", 32),
    "cfg1": ("positions_fmt1_uniform", 16),
    "cfg2": ("positions_fmt1_uniform", 16),
    "cfg3": ("positions_fmt2_uniform", 16),
    "cfg4_2layer": ("positions_fmt2_uniform", 16),
    "cfg4": ("positions_fmt2_uniform", 8),
    "cfg1_mini_tanh": ("positions_fmt1_uniform", 32),
    "cfg3_mini_tanh": ("positions_fmt2_uniform", 32),
    "cfg4_mini_outlier": ("positions_fmt2_uniform", 64),
    "cfg3_mini_polenc": ("positions_fmt2_uniform", 32),
}
# Large batches, recorded in compact form (the logits of the legal moves only, padded to 256 per position, instead of
# all 1858): name -> (net, position set, count).  The batch sizes of the headline measurement.
COMPACT = {
    "cfg4_2layer_b1024": ("cfg4_2layer", "positions_fmt2_uniform", 1024),
    "cfg4_b128": ("cfg4", "positions_fmt2_uniform", 128),
    "cfg5_b128": ("cfg4", "positions_fmt2_split", 128),
}


def read_pos(path):
    b = open(path, "rb").read()
    assert b[:7] == b"LC0POS1"
    n, fmt = np.frombuffer(b[8:16], "<i4")
    off = 16
    masks = np.frombuffer(b, "<u8", n * 112, off).reshape(n, 112); off += n * 112 * 8
    values = np.frombuffer(b, "<f4", n * 112, off).reshape(n, 112); off += n * 112 * 4
    transform = np.frombuffer(b, "<i4", n, off); off += n * 4
    n_legal = np.frombuffer(b, "<i4", n, off); off += n * 4
    legal = np.frombuffer(b, "<i2", n * 256, off).reshape(n, 256)
    return dict(masks=masks, values=values, transform=transform, n_legal=n_legal, legal=legal,
                input_format=np.int32(fmt))


def write_pos(path, p, n):
    with open(path, "wb") as f:
        f.write(b"LC0POS1\0")
        f.write(np.array([n, int(p["input_format"])], "<i4").tobytes())
        f.write(np.ascontiguousarray(p["masks"][:n], "<u8").tobytes())
        f.write(np.ascontiguousarray(p["values"][:n], "<f4").tobytes())
        f.write(np.ascontiguousarray(p["transform"][:n], "<i4").tobytes())
        f.write(np.ascontiguousarray(p["n_legal"][:n], "<i4").tobytes())
        f.write(np.ascontiguousarray(p["legal"][:n], "<i2").tobytes())


def read_out(path):
    b = open(path, "rb").read()
    assert b[:7] == b"LC0OUT1"
    n = int(np.frombuffer(b[8:12], "<i4")[0])
    a = np.frombuffer(b, "<f4", n * (1861 + 256), 12)
    pol = a[:n * 1858].reshape(n, 1858)
    q, d, m = a[n * 1858:n * 1861].reshape(3, n)
    legal_probs = a[n * 1861:].reshape(n, 256)
    return dict(policy=pol, q=q, d=d, m=m, legal_probs=legal_probs)


def main():
    only = set(sys.argv[1:])
    with tempfile.TemporaryDirectory() as tmp:
        sets = {}
        for name, (count, fmt, mix) in POSITION_SETS.items():
            path = os.path.join(tmp, name + ".pos")
            subprocess.check_call([os.path.join(REF, "mkpos"), path, str(count), str(fmt), mix])
            sets[name] = read_pos(path)
            np.savez_compressed(os.path.join(HERE, name + ".npz"), **sets[name])
        for net, (pset, count) in GOLDENS.items():
            if only and net not in only:
                continue
            npath = os.path.join(tmp, net + ".pb.gz")
            mknet.write_net(net, npath)
            ppath = os.path.join(tmp, net + ".pos")
            write_pos(ppath, sets[pset], count)
            opath = os.path.join(tmp, net + ".out")
            subprocess.check_call([os.path.join(REF, "ref_eval"), "blas", npath, ppath, opath, "threads=8"],
                                  stderr=subprocess.DEVNULL)
            out = read_out(opath)
            np.savez_compressed(os.path.join(HERE, "golden_%s.npz" % net), positions=np.array(pset),
                                count=np.int32(count), backend=np.array("blas"), **out)
            os.remove(npath)
            print("golden", net, out["policy"].shape, "q", out["q"][:3], "m", out["m"][:3])
        for name, (net, pset, count) in COMPACT.items():
            if only and name not in only:
                continue
            npath = os.path.join(tmp, net + ".pb.gz")
            mknet.write_net(net, npath)
            ppath = os.path.join(tmp, name + ".pos")
            write_pos(ppath, sets[pset], count)
            opath = os.path.join(tmp, name + ".out")
            subprocess.check_call([os.path.join(REF, "ref_eval"), "blas", npath, ppath, opath, "threads=8"],
                                  stderr=subprocess.DEVNULL)
            out = read_out(opath)
            legal = sets[pset]["legal"][:count].astype(np.int64)
            n_legal = sets[pset]["n_legal"][:count]
            logits = np.take_along_axis(out["policy"], np.clip(legal, 0, 1857), axis=1).astype(np.float32)
            logits[np.arange(256)[None, :] >= n_legal[:, None]] = 0
            np.savez_compressed(os.path.join(HERE, "golden_%s.npz" % name), net=np.array(net), positions=np.array(pset),
                                count=np.int32(count), backend=np.array("blas"), legal_logits=logits, q=out["q"],
                                d=out["d"], m=out["m"], legal_probs=out["legal_probs"])
            os.remove(npath)
            print("golden", name, logits.shape, "q", out["q"][:3], "m", out["m"][:3])


if __name__ == "__main__":
    main()
