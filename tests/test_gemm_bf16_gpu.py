"""The tcgen05 matrix product alone against a float64 product of the same bf16 operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

SHAPES = [  # M, N, K
    (1, 128, 64), (8, 2048, 1536), (8, 1536, 8960), (3, 389, 96), (17, 200, 80),
    (64, 1000, 136), (100, 256, 512), (130, 640, 72), (300, 1536, 1536), (2048, 1792, 1536),
    (33, 151936 // 8, 264),
]


def _ref(x, w, b=None):
    y = x.double() @ w.double().t()
    return y if b is None else y + b.double()


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("bias", [False, True])
def test_product_and_bias(M, N, K, bias):
    from ginfer_b200.ops import gemm_bf16
    g = torch.Generator(device="cpu").manual_seed(M * 7 + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    b = torch.randn(N, generator=g).to(DEV) if bias else None
    want = _ref(x, w, b)
    for split_k, ws in ((None, False), (1, False), (2, False), (4, False), (8, False), (12, False),
                        (3, True)):
        got = gemm_bf16.gemm(x, w, b, torch.bfloat16, split_k=split_k, through_workspace=ws)
        assert got is not None, (split_k, ws)
        torch.testing.assert_close(got.double(), want, atol=2e-2, rtol=1e-2)
    got32 = gemm_bf16.gemm(x, w, b, torch.float32)
    torch.testing.assert_close(got32.double(), want, atol=1e-3, rtol=1e-4)
    gemm_bf16.check_errors()
    # a row does not depend on the other rows of the batch, nor on the tile width they select
    alone = gemm_bf16.gemm(x[:1].contiguous(), w, b, torch.float32, split_k=1)
    full = gemm_bf16.gemm(x, w, b, torch.float32, split_k=1)
    assert torch.equal(alone, full[:1])


@pytest.mark.parametrize("M,I,K", [(8, 8960, 1536), (5, 224, 96), (200, 301, 80), (2048, 512, 256)])
def test_gated_epilogue(M, I, K):
    from ginfer_b200.ops import gemm_bf16
    g = torch.Generator(device="cpu").manual_seed(I)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    gate = (torch.randn(I, K, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    up = (torch.randn(I, K, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    inter = torch.stack([gate, up], dim=1).reshape(2 * I, K).contiguous()
    gg = _ref(x, gate).to(torch.bfloat16).double()      # gate and up are rounded as a product's
    uu = _ref(x, up).to(torch.bfloat16).double()        # output would be, then combined in fp32
    want = gg / (1 + torch.exp(-gg)) * uu
    for split_k, ws in ((None, False), (2, False), (8, False), (5, True)):
        got = gemm_bf16.gemm(x, inter, None, torch.bfloat16, epi=2, split_k=split_k,
                             through_workspace=ws)
        assert got is not None and got.shape == (M, I)
        torch.testing.assert_close(got.double(), want, atol=2e-2, rtol=2e-2)
    gemm_bf16.check_errors()


@pytest.mark.parametrize("M,N,K,split_k", [
    (8, 2048, 1536, 8), (1, 1536, 1536, 8), (16, 392, 512, 4), (13, 1000, 256, 2),   # partials pushed
    (30, 1536, 512, 4), (8, 1536, 1536, 12),
    (8, 1536, 8960, 12), (8, 640, 3072, 4), (40, 512, 1536, 8),                      # partials pulled
])
def test_cluster_split_adds_up_like_the_workspace_split(M, N, K, split_k):
    """The K splits of a cluster are summed in rank order, whether the partials are sent to the
    band owners (K ranges that leave stages of the ring free) or fetched by them: bit for bit what
    the workspace mode gives, which sums in split order too."""
    from ginfer_b200.ops import gemm_bf16
    g = torch.Generator(device="cpu").manual_seed(N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    b = torch.randn(N, generator=g).to(DEV)
    cluster = gemm_bf16.gemm(x, w, b, torch.float32, split_k=split_k)
    through = gemm_bf16.gemm(x, w, b, torch.float32, split_k=split_k, through_workspace=True)
    assert torch.equal(cluster, through)
    torch.testing.assert_close(cluster.double(), _ref(x, w, b), atol=1e-3, rtol=1e-4)
    gemm_bf16.check_errors()


def test_refuses_what_tma_cannot_address():
    from ginfer_b200.ops import gemm_bf16
    x = torch.randn(4, 100, device=DEV).to(torch.bfloat16)        # K = 100: rows of 200 bytes
    w = torch.randn(16, 100, device=DEV).to(torch.bfloat16)
    assert gemm_bf16.gemm(x, w) is None


@pytest.mark.parametrize("M", [1, 8, 16, 17, 32, 64])
@pytest.mark.parametrize("N,K", [(1536, 1536), (1536, 8960), (96, 224), (200, 80), (3584, 18944)])
@pytest.mark.parametrize("bias,gamma_dtype", [(False, None), (True, torch.float32),
                                              (False, torch.bfloat16)])
def test_product_with_residual_and_sums_of_squares(M, N, K, bias, gamma_dtype):
    """``s = resid + x W^T (+ b)``, ``bf16(s * gamma)`` and the partial sums of squares of ``s``,
    whichever way the K range is split."""
    from ginfer_b200.ops import gemm_bf16
    g = torch.Generator(device="cpu").manual_seed(M + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    b = torch.randn(N, generator=g).to(DEV) if bias else None
    gamma = None if gamma_dtype is None else \
        (1 + 0.3 * torch.randn(N, generator=g)).to(gamma_dtype).to(DEV)
    resid = (torch.randn(M, N, generator=g) * 2).to(DEV)
    got = gemm_bf16.gemm(x, w, b, resid=resid, gamma=gamma)
    assert got is not None
    s, scaled, sumsq = got
    want = resid.double() + _ref(x, w, b)
    torch.testing.assert_close(s.double(), want, atol=1e-3, rtol=1e-4)
    assert sumsq.shape == (-(-N // 128) * gemm_bf16.split_k_for(M, N, K), gemm_bf16.sumsq_ld(M))
    torch.testing.assert_close(sumsq[:, :M].double().sum(0), (want ** 2).sum(1), atol=1e-2,
                               rtol=1e-4)
    if gamma is None:
        assert scaled is None
    else:
        assert torch.equal(scaled, (s * gamma.float()).to(torch.bfloat16))
    gemm_bf16.check_errors()


@pytest.mark.parametrize("M", [1, 8, 16, 23, 32, 64])
@pytest.mark.parametrize("N,K,gated", [(2048, 1536, False), (17920, 1536, True), (389, 96, False),
                                       (448, 96, True), (160, 80, False), (151936 // 16, 1536, False)])
def test_product_behind_a_deferred_normalisation(M, N, K, gated):
    """A product over ``s * gamma`` whose accumulator is multiplied by ``1 / rms(s)`` token by
    token, the statistics coming from the product that formed ``s``: against float64, and close
    to the stand-alone norm kernel followed by the plain product."""
    from ginfer_b200 import ops
    from ginfer_b200.ops import gemm_bf16
    g = torch.Generator(device="cpu").manual_seed(M * 3 + N)
    eps = 1e-5
    x0 = torch.randn(M, 64, generator=g).to(torch.bfloat16).to(DEV)
    w0 = (torch.randn(K, 64, generator=g) * 0.3).to(torch.bfloat16).to(DEV)
    r0 = torch.randn(M, K, generator=g).to(DEV)
    gamma = (1 + 0.2 * torch.randn(K, generator=g)).to(DEV)
    prod = gemm_bf16.gemm(x0, w0, None, resid=r0, gamma=gamma)
    assert prod is not None
    s, scaled, sumsq = prod
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    bias = None if gated else torch.randn(N, generator=g).to(DEV)
    out_dtype = torch.float32 if (not gated and N % 5 == 1) else torch.bfloat16
    got = gemm_bf16.gemm(scaled, w, bias, out_dtype, epi=2 if gated else 0,
                         scale=gemm_bf16.RowScale(sumsq, eps))
    assert got is not None
    inv = torch.rsqrt((s.double() ** 2).mean(1, keepdim=True) + eps)
    acc = (scaled.double() @ w.double().t()) * inv
    if gated:
        gate = acc[:, 0::2].to(torch.bfloat16).double()
        up = acc[:, 1::2].to(torch.bfloat16).double()
        want = gate * torch.sigmoid(gate) * up
    else:
        want = acc + bias.double()
    tol = dict(atol=2e-3, rtol=1e-3) if out_dtype == torch.float32 else dict(atol=3e-2, rtol=2e-2)
    torch.testing.assert_close(got.double(), want, **tol)
    zero = torch.zeros((M, K), dtype=torch.bfloat16, device=DEV)
    _, normed = ops.add_rmsnorm(s, zero, gamma, eps)              # bf16, the stand-alone kernel
    plain = gemm_bf16.gemm(normed, w, bias, out_dtype, epi=2 if gated else 0, split_k=1)
    # the two round the operand at different points (before and after the division by rms), so
    # single elements may land on either side of a bf16 rounding step; on the whole they agree
    # (within one rounding step of the operands, 2^-7 relative, on average)
    diff = (got.float() - plain.float()).abs()
    assert float(diff.mean()) < 2.0 ** -7 * max(1.0, float(plain.float().abs().mean()))
    gemm_bf16.check_errors()


@pytest.mark.parametrize("M,N,K,split_k", [(8, 256, 512, 1), (8, 1536, 1536, 8), (40, 384, 2048, 4)])
def test_a_wait_that_runs_out_is_reported_and_the_kernel_returns(M, N, K, split_k):
    """Every wait inside the kernel has a limit.  A build of the same source that leaves out the
    loads of one K block (``-DGF_TEST_SKIP_STAGE``) and polls 3,000 times instead of four million
    makes the MMA issuer's wait for that block run out (role 2), and where a CTA has more K
    blocks than stages also the producer's wait for the stage that is never freed (role 1): the
    kernel must come back, name the role that gave up first in the error word, free its tensor
    memory, and leave the device usable: the regular build then computes the same product
    correctly.  Nothing here faults or hangs: the kernel only stops waiting."""
    from ctypes import c_int, c_void_p

    from ginfer_b200 import ops
    from ginfer_b200.ops import gemm_bf16
    lib = ops.load_library("gemm_bf16", ("GF_SPIN_LIMIT=3000", "GF_TEST_SKIP_STAGE=1"))
    f = lib.gf_gemm_bf16_tc
    f.restype = c_int
    f.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                  c_int, c_int, c_void_p, c_void_p, c_void_p]
    g = torch.Generator(device="cpu").manual_seed(K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    for _ in range(2):                        # twice: tensor memory was freed the first time
        err.zero_()
        rc = f(x.data_ptr(), K, w.data_ptr(), None, out.data_ptr(), N, M, N, K, 0, 0, split_k,
               None, err.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()              # the kernel came back
        blocks = -(-K // 64) // split_k       # K blocks of a CTA; its ring has 6 stages
        assert int(err.item()) in ((2,) if blocks <= 6 else (1, 2))
    got = gemm_bf16.gemm(x, w, None, torch.bfloat16, split_k=split_k)
    torch.testing.assert_close(got.double(), _ref(x, w), atol=2e-2, rtol=1e-2)
    gemm_bf16.check_errors()
