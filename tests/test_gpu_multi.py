"""One batch over several GPUs (b200_multi_*): slices evaluated by per-GPU networks equal one network's results."""
import numpy as np
import pytest

from conftest import load_case
from lc0_b200 import _lib, network

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _check(gpus):
    net, pos, n, g = load_case("cfg4_mini")
    single = network.Network(net, "precision=fp16,max_batch=64")
    multi = network.MultiGpuNetwork(net, "precision=fp16,max_batch=64", gpus=gpus)
    try:
        for count in (n, 37, 2, 1):
            masks, values = np.array(pos["masks"][:count]), np.array(pos["values"][:count])
            want = single.evaluate(masks, values)
            got = multi.evaluate(masks, values)
            # the same kernels on the same rows; tiny batches route some products to the FMA kernel, hence the tolerance
            for k in ("policy", "q", "d", "m"):
                np.testing.assert_allclose(got[k], want[k], atol=2e-3)
        empty = multi.evaluate(np.zeros((0, 112), np.uint64), np.zeros((0, 112), np.float32))
        assert empty["policy"].shape == (0, 1858)
    finally:
        multi.close()
        single.close()


def test_two_networks_on_one_gpu_split_a_batch():
    """The dispatcher's threads, slicing and result placement, with both slices on GPU 0."""
    _check([0, 0])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_split_a_batch():
    _check([0, 1])


def test_bad_gpu_is_reported():
    net, pos, n, g = load_case("cfg3_mini")
    with pytest.raises(_lib.B200Error, match="Invalid GPU Id"):
        network.MultiGpuNetwork(net, "max_batch=8", gpus=[0, 99])
