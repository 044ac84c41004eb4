"""Multi-rank host logic on CPU: batch split and the max-over-ranks reduction over a 2-rank gloo group."""
import os
import subprocess
import sys

import numpy as np

from conftest import ROOT
from lc0_b200 import sharding

WORKER = r"""
import os, sys
sys.path.insert(0, os.environ["B200_ROOT"])
import numpy as np
import torch.distributed as dist
from lc0_b200 import sharding
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
start, stop = sharding.split_batch(1000, world, step=8)[rank]
# each rank "evaluates" its slice: here the slice checksum, so the test can verify coverage without a GPU
local = float(np.arange(1000)[start:stop].sum())
import torch
t = torch.tensor([local], dtype=torch.float64)
dist.all_reduce(t)
slowest = sharding.gather_max(0.5 + rank, dist)
if rank == 0:
    print("RESULT %.1f %.1f %d" % (t.item(), slowest, stop - start))
dist.destroy_process_group()
"""


def test_split_batch_properties():
    for total in (0, 1, 7, 1000, 8192):
        for parts in (1, 2, 3, 8):
            for step in (1, 4, 64):
                sl = sharding.split_batch(total, parts, step)
                assert len(sl) == parts and sl[0][0] == 0 and sl[-1][1] == total
                assert all(a[1] == b[0] for a, b in zip(sl, sl[1:]))
                sizes = [b - a for a, b in sl]
                assert all(s >= 0 for s in sizes) and max(sizes) - min(sizes) < 2 * step
    assert sharding.split_batch(8192, 8) == [(i * 1024, (i + 1) * 1024) for i in range(8)]


def test_two_rank_gloo_group(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, B200_ROOT=ROOT, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29617", str(script)],
                       capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("RESULT")][0].split()
    assert float(line[1]) == float(np.arange(1000).sum())  # the two slices cover the batch exactly once
    assert float(line[2]) == 1.5                            # max over ranks
    assert int(line[3]) == 504


def test_library_slices_agree_with_split_batch():
    """The multi-GPU dispatcher of the library (b200_multi_slice, host code) cuts a batch exactly as split_batch."""
    import ctypes
    from lc0_b200 import _lib
    lib = _lib.load()
    for total, parts in ((10, 4), (8192, 8), (3, 8), (0, 2), (1025, 2), (1, 1), (4097, 3)):
        want = sharding.split_batch(total, parts)
        got = []
        for i in range(parts):
            b, c = ctypes.c_int(), ctypes.c_int()
            lib.b200_multi_slice(total, parts, i, ctypes.byref(b), ctypes.byref(c))
            got.append((b.value, b.value + c.value))
        assert got == want
