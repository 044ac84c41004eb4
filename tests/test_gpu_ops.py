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


# ---- folded-LayerNorm epilogues of the tensor-core product (b200_op_gemm_ex) -------------------------------------
def _desc(**kw):
    d = _lib.GemmDesc()
    d.scale, d.alpha = 1.0, 1.0
    for k, v in kw.items():
        setattr(d, k, v.data_ptr() if hasattr(v, "data_ptr") else v)
    return d


def _planted_rows(M):
    """Row classes of the epilogue tests: rows whose mean is many standard deviations away from zero, rows with one
    channel at 3e3 or 1e4, and ordinary rows."""
    r = np.arange(M)
    return {"shifted": r[r % 7 == 3], "outlier3e3": r[r % 11 == 5], "outlier1e4": r[r % 13 == 8]}


def _fold(W, b, gamma, beta, dt):
    """What the loader does for a product that consumes a folded LayerNorm: W * gamma rounded to the storage type,
    its row sums, and beta . W^T + b."""
    Wg = (W * gamma[None, :]).to(dt)
    colsum = Wg.float().sum(dim=1).contiguous()
    bias = (b.double() + (W.double() * beta.double()[None, :]).sum(dim=1)).float().contiguous()
    return Wg.contiguous(), colsum, bias


@pytest.mark.parametrize("prec,M,shift", [(1, 65536, 100.0), (2, 8192 + 77, 10.0)])
def test_folded_layer_norm_epilogues_against_oracle(lib, prec, M, shift):
    """The three epilogue forms an encoder layer uses, chained as in the layer, at the row count of batch 1024:
      1. u  = alpha * (A0 W0^T + b0) + R            with per-row (sum, sum of squares) of u accumulated by atomics
      2. h  = relu2(LN(u) W1^T + b1)                LayerNorm folded: row scale and rank-1 correction from the statistics
      3. u2 = alpha * (h W2^T + b2) + LN(u)         the residual normalised on the fly, statistics of u2 again
    against oracle.fc / oracle.layer_norm (fully_connected_layer.cc:50-106, backends/blas/encoder.h:29-78) on a
    sample of rows that contains every planted row class.  The row statistics are sums of the unrounded outputs while
    the consumer reads the rounded ones, so bf16 (spacing 0.5 at 100) gets a smaller row shift than fp16."""
    dt = DT[prec]
    E, F = 1024, 1536
    alpha, eps_ln = 0.43, 1e-3
    g = torch.Generator(device="cuda").manual_seed(M + prec)
    rnd = lambda *s: torch.randn(*s, device="cuda", generator=g)
    A0 = (rnd(M, E) * 0.5).to(dt)
    W0 = (rnd(E, E) * E ** -0.5).to(dt)
    b0 = rnd(E) * 0.1
    R = rnd(M, E)
    rows = _planted_rows(M)
    R[torch.from_numpy(rows["shifted"]).cuda()] += shift
    R[torch.from_numpy(rows["outlier3e3"]).cuda(), 5] = 3000.0
    R[torch.from_numpy(rows["outlier1e4"]).cuda(), 700] = -10000.0
    R = R.to(dt)
    gamma = 1 + rnd(E) * 0.1
    beta = rnd(E) * 0.1
    W1 = rnd(F, E) * E ** -0.5
    b1 = rnd(F) * 0.1
    W2 = (rnd(E, F) * F ** -0.5).to(dt)
    b2 = rnd(E) * 0.1
    W1g, cs1, b1f = _fold(W1, b1, gamma, beta, dt)

    u = torch.zeros(M, E, dtype=dt, device="cuda")
    st1 = torch.zeros(M, 2, device="cuda", dtype=torch.float64)
    _lib.check(lib.b200_op_gemm_ex(_desc(A=A0, W=W0, bias=b0, C=u, M=M, N=E, K=E, precision=prec, alpha=alpha,
                                         res=R, out_stats=st1), None))
    h = torch.zeros(M, F, dtype=dt, device="cuda")
    _lib.check(lib.b200_op_gemm_ex(_desc(A=u, W=W1g, bias=b1f, C=h, M=M, N=F, K=E, precision=prec,
                                         activation=oracle.ACT_RELU_2, a_stats=st1, colsum=cs1, a_inv_c=1.0 / E,
                                         a_eps=eps_ln), None))
    u2 = torch.zeros(M, E, dtype=dt, device="cuda")
    st2 = torch.zeros(M, 2, device="cuda", dtype=torch.float64)
    _lib.check(lib.b200_op_gemm_ex(_desc(A=h, W=W2, bias=b2, C=u2, M=M, N=E, K=F, precision=prec, alpha=alpha,
                                         res=u, res_stats=st1, res_gamma=gamma, res_beta=beta, res_inv_c=1.0 / E,
                                         res_eps=eps_ln, out_stats=st2), None))
    torch.cuda.synchronize()

    rng = np.random.default_rng(7)
    sample = np.unique(np.concatenate([rows["shifted"][:96], rows["outlier3e3"][:64], rows["outlier1e4"][:64],
                                       rng.integers(0, M, 256), [0, M - 1]]))
    sel = torch.from_numpy(sample).cuda()
    f = lambda t: (t if t.dtype == torch.float64 else t.float()).cpu().numpy()
    rt = 2.0 ** -10 if prec == 1 else 2.0 ** -7  # output rounding of the storage type
    # 1: product + plain residual + statistics
    u_ref = alpha * oracle.fc(f(A0[sel]), f(W0).reshape(-1), f(b0), oracle.ACT_NONE, E) + f(R[sel])
    assert np.all(np.abs(f(u[sel]) - u_ref) <= rt * np.abs(u_ref) + 2e-3)
    s_ref = np.stack([u_ref.sum(-1, dtype=np.float64), (u_ref.astype(np.float64) ** 2).sum(-1)], 1)
    mag = np.stack([np.abs(u_ref).sum(-1, dtype=np.float64), s_ref[:, 1]], 1)  # what the fp32 partial sums add up
    assert np.all(np.abs(f(st1[sel]) - s_ref) <= 2e-5 * mag + 1e-3)
    # 2: folded LayerNorm of the stored (rounded) u, two-pass in the oracle
    un = f(u[sel])
    x = oracle.layer_norm(un, 1.0, None, np.ones(E, np.float32), np.zeros(E, np.float32), eps_ln)
    h_ref = oracle.fc(x, f(W1g).reshape(-1), f(b1f), oracle.ACT_RELU_2, F)
    # Rows shifted by `shift` standard deviations: the folded form computes LN(u) W^T as rstd * (u W'^T - mean * colsum),
    # two terms of size |mean| * |colsum| that cancel; the tensor core accumulates the first one at that size, so the
    # pre-activation loses about 1e-4 * shift (fp16; more in bf16, whose statistics are also sums of the unrounded
    # values while the product reads the rounded ones), and relu^2 turns it into 2 * sqrt(h) times that.
    is_shifted = np.isin(sample, rows["shifted"])[:, None]
    per_shift = 2e-4 if prec == 1 else 1e-3

    def worst(got, ref, floor):
        extra = np.where(is_shifted, per_shift * shift * (1 + 2 * np.sqrt(np.abs(ref))), 0.0)
        err = np.abs(got - ref) - (rt * np.abs(ref) + floor + extra)
        r, c = np.unravel_index(err.argmax(), err.shape)
        cls = [k for k, v in rows.items() if sample[r] in v] or ["ordinary"]
        return err.max(), "excess %.3g at row %d (%s) column %d: got %.6g, reference %.6g" % (
            err.max(), sample[r], "+".join(cls), c, got[r, c], ref[r, c])

    e, msg = worst(f(h[sel]), h_ref, 3e-3)
    assert e <= 0, "folded LayerNorm product: " + msg
    # 3: residual normalised on the fly
    ln_u = oracle.layer_norm(un, 1.0, None, f(gamma), f(beta), eps_ln)
    u2_ref = alpha * oracle.fc(f(h[sel]), f(W2).reshape(-1), f(b2), oracle.ACT_NONE, E) + ln_u
    e, msg = worst(f(u2[sel]), u2_ref, 3e-3)
    assert e <= 0, "normalised residual: " + msg
    s2_ref = np.stack([u2_ref.sum(-1, dtype=np.float64), (u2_ref.astype(np.float64) ** 2).sum(-1)], 1)
    mag2 = np.stack([np.abs(u2_ref).sum(-1, dtype=np.float64), s2_ref[:, 1]], 1)
    # u2_ref is built from the rounded h and u, the kernel's sums from its own unrounded values: the storage
    # type's rounding, not the summation, bounds the difference
    assert np.all(np.abs(f(st2[sel]) - s2_ref) <= 4 * rt * mag2 + 1e-2)


@pytest.mark.parametrize("whole_tiles", [0, 1])
def test_second_output_of_the_pair_kernel_with_folded_input(lib, whole_tiles):
    """Q, K, V and the smolgen compression from one launch (columns from n_split on go to a second matrix through a
    narrow last tile), with the LayerNorm of the input folded in, at the row count of batch 1024."""
    M, E, N, hc = 65536, 1024, 3072, 32
    g = torch.Generator(device="cuda").manual_seed(11)
    rnd = lambda *s: torch.randn(*s, device="cuda", generator=g)
    u = (rnd(M, E) * 2 + 0.5).half()
    gamma, beta = 1 + rnd(E) * 0.1, rnd(E) * 0.1
    W = rnd(N + hc, E) * E ** -0.5
    b = torch.cat([rnd(N) * 0.1, torch.zeros(hc, device="cuda")])
    Wg, cs, bf = _fold(W, b, gamma, beta, torch.float16)
    uf = u.double()
    stats = torch.stack([uf.sum(1), (uf * uf).sum(1)], 1).contiguous()
    C = torch.zeros(M, N, dtype=torch.float16, device="cuda")
    C2 = torch.zeros(M, hc, dtype=torch.float16, device="cuda")
    _lib.check(lib.b200_op_gemm_ex(_desc(A=u, W=Wg, bias=bf, C=C, M=M, N=N + hc, K=E, precision=1, a_stats=stats,
                                         colsum=cs, a_inv_c=1.0 / E, a_eps=1e-3, C2=C2, ldc2=hc, n_split=N,
                                         whole_tiles=whole_tiles), None))
    torch.cuda.synchronize()
    sample = np.unique(np.concatenate([np.random.default_rng(3).integers(0, M, 300), [0, 127, 128, M - 129, M - 1]]))
    sel = torch.from_numpy(sample).cuda()
    f = lambda t: t.float().cpu().numpy()
    x = oracle.layer_norm(f(u[sel]), 1.0, None, np.ones(E, np.float32), np.zeros(E, np.float32), 1e-3)
    ref = oracle.fc(x, f(Wg).reshape(-1), f(bf), oracle.ACT_NONE, N + hc)
    got = np.concatenate([f(C[sel]), f(C2[sel])], 1)
    assert np.all(np.abs(got - ref) <= 2.0 ** -10 * np.abs(ref) + 3e-3)


def test_gemm_ex_rejects_inconsistent_descriptions(lib):
    a = torch.zeros(256, 64, dtype=torch.float16, device="cuda")
    st = torch.zeros(256, 2, device="cuda", dtype=torch.float64)
    assert lib.b200_op_gemm_ex(_desc(A=a, W=a, C=a, M=256, N=64, K=64, precision=0), None) == _lib.ERR_UNSUPPORTED
    assert lib.b200_op_gemm_ex(_desc(A=a, W=a, C=a, M=256, N=64, K=64, precision=1, a_stats=st), None) == \
        _lib.ERR_UNSUPPORTED  # statistics without column sums
    assert lib.b200_op_gemm_ex(_desc(A=a, W=a, C=a, M=256, N=64, K=64, precision=1, C2=a, ldc2=64, n_split=32),
                               None) == _lib.ERR_UNSUPPORTED  # too small for the kernel that has a second output
    assert lib.b200_op_gemm_ex(None, None) == _lib.ERR_INVALID
