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
    for split_k, ws in ((None, False), (1, False), (2, False), (4, False), (8, False), (3, True)):
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


def test_refuses_what_tma_cannot_address():
    from ginfer_b200.ops import gemm_bf16
    x = torch.randn(4, 100, device=DEV).to(torch.bfloat16)        # K = 100: rows of 200 bytes
    w = torch.randn(16, 100, device=DEV).to(torch.bfloat16)
    assert gemm_bf16.gemm(x, w) is None
