"""The allocation-free attention-policy operator against the regular one.

Engines that call the backend from search threads, and hosts whose own pool owns all free device memory,
cannot allocate scratch per call; b200_op_policy_attention_static keeps its scratch inside the library.
This file sorts last on purpose: a run that stops at the first failure has then already run everything else.
"""
import numpy as np
import pytest

from lc0_b200 import _lib

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

DT = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}


def _both(lib, prec, n, dm, seed, stream=None):
    torch.manual_seed(seed)
    q = torch.randn(n, 64, dm, device="cuda").to(DT[prec])
    k = torch.randn(n, 64, dm, device="cuda").to(DT[prec])
    w4 = torch.randn(4, dm, device="cuda") * 0.1
    scratch = torch.empty(n, 4096, device="cuda")
    want = torch.zeros(n, 1858, device="cuda")
    got = torch.full((n, 1858), 7.0, device="cuda")
    torch.cuda.synchronize()  # the inputs were produced on torch's stream
    st = stream.cuda_stream if stream is not None else None
    _lib.check(lib.b200_op_policy_attention(q.data_ptr(), k.data_ptr(), w4.data_ptr(), dm, n, scratch.data_ptr(),
                                            want.data_ptr(), prec, st))
    _lib.check(lib.b200_op_policy_attention_static(q.data_ptr(), k.data_ptr(), w4.data_ptr(), dm, n,
                                                   got.data_ptr(), prec, st))
    torch.cuda.synchronize()
    return got.cpu().numpy(), want.cpu().numpy()


@pytest.mark.parametrize("prec", [0, 1])
def test_static_scratch_matches_regular_operator_twice(lib, prec):
    # two calls in a row: the second must not be disturbed by what the first left in the shared scratch
    for seed, n, dm in ((1, 37, 128), (2, 5, 64)):
        got, want = _both(lib, prec, n, dm, seed)
        assert np.abs(got - want).max() <= 2e-4 * max(1.0, np.abs(want).max())
        assert np.abs(want).max() > 0.1


def test_static_scratch_on_a_non_blocking_stream_and_bf16(lib):
    """A caller stream that does not synchronise with the default stream (the first call's table upload must have
    landed before the kernels run there), and bf16 storage."""
    stream = torch.cuda.Stream()  # torch's side streams are created non-blocking
    for seed, n, dm in ((3, 64, 96), (4, 9, 256)):
        got, want = _both(lib, 2, n, dm, seed, stream)
        assert np.abs(got - want).max() <= 2e-4 * max(1.0, np.abs(want).max())
        assert np.abs(want).max() > 0.1


def test_static_scratch_limit_and_empty(lib):
    assert lib.b200_op_policy_attention_static(None, None, None, 64, 0, None, 0, None) == _lib.OK
    x = torch.zeros(8, device="cuda")
    rc = lib.b200_op_policy_attention_static(x.data_ptr(), x.data_ptr(), x.data_ptr(), 64, 257, x.data_ptr(), 0, None)
    assert rc == _lib.ERR_INVALID
    assert b"exceed" in lib.b200_last_error()
