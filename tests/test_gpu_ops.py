"""Stand-alone operator entry points of the C ABI against the oracle's restatements."""
import numpy as np
import pytest

from lc0_b200 import _lib
from oracle import oracle

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

DT = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}


@pytest.mark.parametrize("prec", [0, 1, 2])
@pytest.mark.parametrize("n", [1, 3, 64, 257])
def test_expand_planes_bit_exact(lib, prec, n):
    rng = np.random.default_rng(n)
    masks = rng.integers(0, 2 ** 63, size=(n, 112), dtype=np.uint64) * np.uint64(2) + rng.integers(0, 2, size=(n, 112)).astype(np.uint64)
    values = rng.choice(np.array([1.0, 0.5, 0.25, 3.0, 99.0], np.float32), size=(n, 112))
    want = oracle.expand_planes(masks, values)
    dm = torch.from_numpy(masks.view(np.int64)).cuda()
    dv = torch.from_numpy(values).cuda()
    out = torch.zeros(n, 112, 64, dtype=DT[prec], device="cuda")
    _lib.check(lib.b200_op_expand_planes(dm.data_ptr(), dv.data_ptr(), n, out.data_ptr(), prec, None))
    torch.cuda.synchronize()
    assert np.array_equal(out.float().cpu().numpy(), want)  # all test values are exact in every type


def test_expand_planes_empty(lib):
    _lib.check(lib.b200_op_expand_planes(None, None, 0, None, 0, None))


@pytest.mark.parametrize("prec", [1, 2])
@pytest.mark.parametrize("shape", [(128, 64, 64), (64, 256, 512), (1000, 1024, 1024), (333, 200, 72),
                                   (8192, 3072, 1024), (4096, 1024, 1536), (130, 4096, 256), (2048, 32, 1024),
                                   # CTA-pair kernel with row / column tails (narrow last MMA tile) and few k-blocks
                                   # (four epilogue groups)
                                   (5000, 1312, 256), (3000, 2000, 1024), (2560, 1096, 320),
                                   # a last wave of at most half the CTA pairs: computed as half-width tiles
                                   (16384, 1024, 1024), (19200, 512, 256), (9600, 1024, 576)])
@pytest.mark.parametrize("act", [oracle.ACT_NONE, oracle.ACT_RELU_2, oracle.ACT_MISH])
def test_tensor_core_gemm(lib, prec, shape, act):
    M, N, K = shape
    torch.manual_seed(M + N + K)
    A = (torch.randn(M, K, device="cuda") * 0.5).to(DT[prec])
    W = (torch.randn(N, K, device="cuda") * (K ** -0.5)).to(DT[prec])
    b = torch.randn(N, device="cuda") * 0.1
    C = torch.zeros(M, N, dtype=DT[prec], device="cuda")
    _lib.check(lib.b200_op_gemm(A.data_ptr(), W.data_ptr(), b.data_ptr(), C.data_ptr(), M, N, K, act, prec, 1, None))
    torch.cuda.synchronize()
    ref = oracle.fc(A.float().cpu().numpy(), W.float().cpu().numpy().reshape(-1), b.cpu().numpy(), act, N)
    got = C.float().cpu().numpy()
    eps = 2.0 ** -10 if prec == 1 else 2.0 ** -7  # output rounding of the storage type
    assert np.all(np.abs(got - ref) <= eps * np.abs(ref) + 2e-3)


@pytest.mark.parametrize("prec", [0, 1, 2])
def test_fma_gemm(lib, prec):
    M, N, K = 77, 130, 45
    torch.manual_seed(0)
    A = (torch.randn(M, K, device="cuda")).to(DT[prec])
    W = (torch.randn(N, K, device="cuda") * 0.2).to(DT[prec])
    b = torch.randn(N, device="cuda")
    C = torch.zeros(M, N, dtype=DT[prec], device="cuda")
    _lib.check(lib.b200_op_gemm(A.data_ptr(), W.data_ptr(), b.data_ptr(), C.data_ptr(), M, N, K, oracle.ACT_SWISH, prec, 0, None))
    torch.cuda.synchronize()
    ref = oracle.fc(A.float().cpu().numpy(), W.float().cpu().numpy().reshape(-1), b.cpu().numpy(), oracle.ACT_SWISH, N)
    tol = {0: 1e-5, 1: 2e-3, 2: 1.6e-2}[prec]
    assert np.abs(C.float().cpu().numpy() - ref).max() <= tol * max(1.0, np.abs(ref).max())


def test_gemm_tc_rejects_fp32(lib):
    assert lib.b200_op_gemm(None, None, None, None, 128, 128, 64, 3, 0, 1, None) == _lib.ERR_UNSUPPORTED


@pytest.mark.parametrize("prec", [0, 1, 2])
@pytest.mark.parametrize("C", [64, 256, 1024, 8192])
def test_layer_norm(lib, prec, C):
    rows = 130
    torch.manual_seed(C)
    x = torch.randn(rows, C, device="cuda").to(DT[prec])
    skip = torch.randn(rows, C, device="cuda").to(DT[prec])
    gam = torch.randn(C, device="cuda") * 0.1 + 1
    bet = torch.randn(C, device="cuda") * 0.1
    out = torch.zeros(rows, C, dtype=DT[prec], device="cuda")
    _lib.check(lib.b200_op_layer_norm(out.data_ptr(), x.data_ptr(), skip.data_ptr(), gam.data_ptr(), bet.data_ptr(),
                                      rows, C, 0.43, 1e-3, prec, None))
    torch.cuda.synchronize()
    ref = oracle.layer_norm(x.float().cpu().numpy(), 0.43, skip.float().cpu().numpy(), gam.cpu().numpy(),
                            bet.cpu().numpy(), 1e-3)
    tol = {0: 2e-5, 1: 4e-3, 2: 3e-2}[prec]
    assert np.abs(out.float().cpu().numpy() - ref).max() <= tol


def _policy_reference(q, k, w4):
    """Attention-policy tail restated with the oracle's table (network_blas.cc:850-914)."""
    from oracle import tables
    n, _, dm = q.shape
    logits = np.matmul(q, k.transpose(0, 2, 1)) / np.sqrt(np.float32(dm))
    off = np.einsum("njk,ik->nij", k[:, 56:64, :], w4)
    off[:, :3, :] += off[:, 3:4, :]
    promo = logits[:, 48:56, 56:64][:, :, :, None] + off[:, :3, :].transpose(0, 2, 1)[:, None, :, :]
    raw = np.concatenate([logits.reshape(n, 4096), promo.reshape(n, 192)], axis=1)
    pmap = tables.attn_policy_map()
    out = np.zeros((n, 1858), np.float32)
    out[:, pmap[pmap >= 0]] = raw[:, pmap >= 0]
    return out


@pytest.mark.parametrize("prec", [0, 1])
@pytest.mark.parametrize("n,dm", [(1, 64), (5, 96), (33, 256)])
def test_policy_attention_op(lib, prec, n, dm):
    torch.manual_seed(n * dm)
    q = torch.randn(n, 64, dm, device="cuda").to(DT[prec])
    k = torch.randn(n, 64, dm, device="cuda").to(DT[prec])
    w4 = torch.randn(4, dm, device="cuda") * 0.1
    scratch = torch.empty(n, 4096, device="cuda")
    pol = torch.zeros(n, 1858, device="cuda")
    _lib.check(lib.b200_op_policy_attention(q.data_ptr(), k.data_ptr(), w4.data_ptr(), dm, n, scratch.data_ptr(),
                                            pol.data_ptr(), prec, None))
    torch.cuda.synchronize()
    want = _policy_reference(q.float().cpu().numpy(), k.float().cpu().numpy(), w4.cpu().numpy())
    assert np.abs(pol.cpu().numpy() - want).max() <= 2e-4 * max(1.0, np.abs(want).max())


def _attention_reference(qkv, bias, n, heads, depth):
    """softmax(Q K^T / sqrt(depth) + bias) V per (position, head) in fp32 (network_blas.cc:352-439)."""
    e = heads * depth
    x = qkv.float().reshape(n, 64, 3, heads, depth)
    q, k, v = (x[:, :, i].permute(0, 2, 1, 3) for i in range(3))  # [n][heads][64][depth]
    s = torch.matmul(q, k.transpose(-1, -2)) / depth ** 0.5
    if bias is not None:
        s = s + bias.float().reshape(n, heads, 64, 64)
    p = torch.softmax(s, dim=-1)
    return torch.matmul(p, v).permute(0, 2, 1, 3).reshape(n * 64, e)


@pytest.mark.parametrize("variant", [0, 1])
@pytest.mark.parametrize("prec", [1, 2])
@pytest.mark.parametrize("n,heads,depth,with_bias", [(1, 4, 32, True), (7, 32, 32, True), (3, 8, 64, False),
                                                     (150, 8, 32, True), (40, 6, 64, True), (2, 1, 32, False)])
def test_attention_op(lib, variant, prec, n, heads, depth, with_bias):
    """Both attention kernels against an fp32 reference on the fused Q|K|V layout the network uses; the
    persistent TMA kernel (variant 1) walks several items per CTA at the larger sizes."""
    torch.manual_seed(n * heads + depth)
    e = heads * depth
    qkv = torch.randn(n * 64, 3 * e, device="cuda").to(DT[prec])
    bias = (torch.randn(n, heads, 64, 64, device="cuda") * 2).to(DT[prec]) if with_bias else None
    out = torch.zeros(n * 64, e, device="cuda", dtype=DT[prec])
    esz = 2
    _lib.check(lib.b200_op_attention(qkv.data_ptr(), qkv.data_ptr() + e * esz, qkv.data_ptr() + 2 * e * esz, 3 * e,
                                     bias.data_ptr() if with_bias else None, out.data_ptr(), e, n, heads, depth, prec,
                                     variant, None))
    torch.cuda.synchronize()
    want = _attention_reference(qkv, bias, n, heads, depth)
    tol = 4e-3 if prec == 1 else 3e-2  # probabilities and outputs are rounded to 16 bits (11 / 8 significant bits)
    assert (out.float() - want).abs().max().item() <= tol * max(1.0, want.abs().max().item())


def test_attention_op_variants_agree(lib):
    """The FMA kernel and the persistent TMA kernel on the same 16-bit inputs."""
    torch.manual_seed(5)
    n, heads, depth = 64, 32, 32
    e = heads * depth
    qkv = torch.randn(n * 64, 3 * e, device="cuda").half()
    bias = torch.randn(n, heads, 64, 64, device="cuda").half()
    outs = []
    for variant in (0, 1):
        out = torch.zeros(n * 64, e, device="cuda", dtype=torch.float16)
        _lib.check(lib.b200_op_attention(qkv.data_ptr(), qkv.data_ptr() + e * 2, qkv.data_ptr() + 4 * e, 3 * e,
                                         bias.data_ptr(), out.data_ptr(), e, n, heads, depth, 1, variant, None))
        outs.append(out.float())
    torch.cuda.synchronize()
    assert (outs[0] - outs[1]).abs().max().item() <= 4e-3


def test_attention_op_rejects_fp32_tensor_core_variants(lib):
    assert lib.b200_op_attention(None, None, None, 96, None, None, 32, 0, 1, 32, 0, 1, None) == _lib.ERR_UNSUPPORTED
