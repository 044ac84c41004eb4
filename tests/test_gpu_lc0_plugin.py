"""The backend driven by lc0 itself: the reference's factory, loader and `check` decorator.

Uses oracle/_ref/ref_eval and lc0_ref (the reference's sources compiled with the plug-in TU
lc0_b200/adapter/network_b200.cc by `python oracle/build_ref.py --adapter`); skipped when they are absent.
"""
import os
import subprocess

import numpy as np
import pytest

from conftest import ROOT, load_case
from lc0_b200 import mknet

pytestmark = pytest.mark.gpu
REF = os.path.join(ROOT, "oracle", "_ref")


def _has_plugin():
    exe = os.path.join(REF, "lc0_ref")
    if not os.path.exists(exe):
        return False
    r = subprocess.run([exe, "backendbench", "--help"], capture_output=True, text=True)
    return "b200" in r.stdout + r.stderr


needs_plugin = pytest.mark.skipif(not _has_plugin(), reason="lc0 with the b200 plug-in is not built")


def _write_pos(path, pos, n):
    with open(path, "wb") as f:
        f.write(b"LC0POS1\0")
        f.write(np.array([n, int(pos["input_format"])], "<i4").tobytes())
        f.write(np.ascontiguousarray(pos["masks"][:n], "<u8").tobytes())
        f.write(np.ascontiguousarray(pos["values"][:n], "<f4").tobytes())
        f.write(np.zeros(2 * n, "<i4").tobytes())
        f.write(np.full((n, 256), -1, "<i2").tobytes())


@needs_plugin
@pytest.mark.parametrize("name", ["cfg4_mini", "cfg2_mini"])
def test_registered_backend_through_lc0_factory(tmp_path, name):
    net, pos, n, g = load_case(name)
    npath, ppath, opath = str(tmp_path / "n.pb.gz"), str(tmp_path / "p.pos"), str(tmp_path / "o.bin")
    mknet.write_net(name, npath)
    _write_pos(ppath, pos, n)
    r = subprocess.run([os.path.join(REF, "ref_eval"), "b200-fp32", npath, ppath, opath, "max_batch=64"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    raw = np.fromfile(opath, "<f4", offset=12)
    pol = raw[:n * 1858].reshape(n, 1858)
    q, d, m = raw[n * 1858:n * 1861].reshape(3, n)
    scale = np.abs(g["policy"]).max()
    assert np.abs(pol - g["policy"]).max() <= 1e-5 * scale
    assert np.abs(q - g["q"]).max() <= 1e-5 and np.abs(d - g["d"]).max() <= 1e-5
    assert np.abs(m - g["m"]).max() <= 1e-5 * max(1.0, np.abs(g["m"]).max())


@needs_plugin
def test_unknown_option_is_fatal_like_other_backends(tmp_path):
    npath, ppath = str(tmp_path / "n.pb.gz"), str(tmp_path / "p.pos")
    mknet.write_net("cfg3_mini", npath)
    net, pos, n, g = load_case("cfg3_mini")
    _write_pos(ppath, pos, 2)
    r = subprocess.run([os.path.join(REF, "ref_eval"), "b200", npath, ppath, "-", "gpu=99"], capture_output=True, text=True)
    assert r.returncode != 0 and "Invalid GPU Id" in r.stderr


@needs_plugin
def test_lc0_backendbench_and_check_decorator(tmp_path):
    npath = str(tmp_path / "n.pb.gz")
    mknet.write_net("cfg3_mini", npath)
    exe = os.path.join(REF, "lc0_ref")
    r = subprocess.run([exe, "backendbench", "--weights=" + npath, "--backend=check",
                        "--backend-opts=mode=check,freq=1.0,atol=1e-4,rtol=1e-3,(backend=b200-fp32),(backend=blas)",
                        "--batches=2", "--start-batch-size=8", "--max-batch-size=16", "--batch-step=8"],
                       capture_output=True, text=True, timeout=300)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-2000:]
    assert "Check passed" in out or "passed" in out.lower(), out[-2000:]


def _search(exe, npath, backend, opts, nodes=400, positions=3, extra=()):
    cmd = [exe, "benchmark", "--weights=" + npath, "--backend=" + backend, "--nodes=%d" % nodes, "--threads=1",
           "--num-positions=%d" % positions] + list(extra)
    if opts:
        cmd.append("--backend-opts=" + opts)
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-2000:]
    best = [l.split()[1] for l in out.splitlines() if l.startswith("bestmove")]
    assert len(best) == positions, out[-2000:]
    return best


@needs_plugin
def test_native_backend_searches_like_the_wrapped_network(tmp_path):
    """lc0's own single-threaded search over the native Backend ("b200-native": position encoding and legal-move
    softmax on the device, compact return) picks the same moves as over the Network adapter behind lc0's wrapper
    (host encoder, host softmax)."""
    npath = str(tmp_path / "n.pb.gz")
    mknet.write_net("cfg4_mini", npath)
    exe = os.path.join(REF, "lc0_ref")
    wrapped = _search(exe, npath, "b200", "")
    native = _search(exe, npath, "b200-native", "")  # game histories go to the device, planes are produced there
    assert native == wrapped
    host_encoded = _search(exe, npath, "b200-native", "device_encode=false")
    assert host_encoded == wrapped
    native32 = _search(exe, npath, "b200-native", "precision=fp32")
    wrapped32 = _search(exe, npath, "b200-fp32", "")
    assert native32 == wrapped32


@needs_plugin
def test_native_backend_backendbench_and_options(tmp_path):
    npath = str(tmp_path / "n.pb.gz")
    mknet.write_net("cfg3_mini", npath)
    exe = os.path.join(REF, "lc0_ref")
    r = subprocess.run([exe, "backendbench", "--weights=" + npath, "--backend=b200-native",
                        "--backend-opts=max_batch=2048", "--batches=2", "--start-batch-size=512",
                        "--max-batch-size=1024", "--batch-step=256"], capture_output=True, text=True, timeout=300)
    out = r.stdout + r.stderr
    assert r.returncode == 0 and "1024" in out, out[-2000:]
    r = subprocess.run([exe, "backendbench", "--weights=" + npath, "--backend=b200-native",
                        "--backend-opts=precision=fp64", "--batches=1"], capture_output=True, text=True, timeout=300)
    assert "unknown precision" in r.stdout + r.stderr


@needs_plugin
def test_mux_backend_matches_the_reference_outputs_and_searches_like_b200(tmp_path):
    """"b200-mux" (every computation goes through the library's batch aggregator): the recorded reference outputs in
    fp32, the same moves as "b200" in lc0's single-threaded search, and lc0's multi-threaded search runs over it."""
    net, pos, n, g = load_case("cfg4_mini")
    npath, ppath, opath = str(tmp_path / "n.pb.gz"), str(tmp_path / "p.pos"), str(tmp_path / "o.bin")
    mknet.write_net("cfg4_mini", npath)
    _write_pos(ppath, pos, n)
    r = subprocess.run([os.path.join(REF, "ref_eval"), "b200-mux", npath, ppath, opath, "max_batch=64,precision=fp32"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    raw = np.fromfile(opath, "<f4", offset=12)
    pol = raw[:n * 1858].reshape(n, 1858)
    q = raw[n * 1858:n * 1859]
    assert np.abs(pol - g["policy"]).max() <= 1e-5 * np.abs(g["policy"]).max()
    assert np.abs(q - g["q"]).max() <= 1e-5
    exe = os.path.join(REF, "lc0_ref")
    # the same minibatch size for both: lc0 otherwise takes each backend's own recommendation, which shapes the search
    mb = ["--minibatch-size=32"]
    assert _search(exe, npath, "b200-mux", "", extra=mb) == _search(exe, npath, "b200", "", extra=mb)
    r = subprocess.run([exe, "benchmark", "--weights=" + npath, "--backend=b200-mux", "--backend-opts=mux_wait_us=100",
                        "--nodes=2000", "--threads=4", "--num-positions=2"], capture_output=True, text=True, timeout=600)
    out = r.stdout + r.stderr
    assert r.returncode == 0 and out.count("bestmove") == 2, out[-2000:]
    r = subprocess.run([exe, "backendbench", "--weights=" + npath, "--backend=b200-mux",
                        "--backend-opts=precision=fp64", "--batches=1"], capture_output=True, text=True, timeout=300)
    assert "precision must be" in r.stdout + r.stderr


@needs_plugin
def test_multi_gpu_backend_matches_the_reference_outputs(tmp_path):
    """"b200-multi" (the batch cut into one slice per GPU by the library); with one GPU in the box both slices run on
    it (gpus=1 is the degenerate case, two networks on GPU 0 are covered by tests/test_gpu_multi.py)."""
    import torch
    count = min(2, torch.cuda.device_count())
    net, pos, n, g = load_case("cfg4_mini")
    npath, ppath, opath = str(tmp_path / "n.pb.gz"), str(tmp_path / "p.pos"), str(tmp_path / "o.bin")
    mknet.write_net("cfg4_mini", npath)
    _write_pos(ppath, pos, n)
    r = subprocess.run([os.path.join(REF, "ref_eval"), "b200-multi", npath, ppath, opath,
                        "max_batch=64,precision=fp32,gpus=%d" % count], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    raw = np.fromfile(opath, "<f4", offset=12)
    pol = raw[:n * 1858].reshape(n, 1858)
    q = raw[n * 1858:n * 1859]
    assert np.abs(pol - g["policy"]).max() <= 1e-5 * np.abs(g["policy"]).max()
    assert np.abs(q - g["q"]).max() <= 1e-5
