"""The persistent tcgen05 product for many tokens alone against a float64 product of the same bf16
operands: tiles that are cut by M, N and K, more tiles than CTAs (both accumulators and every
ring stage are used again), bias, fp32 output, the gated epilogue."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

SHAPES = [  # M, N, K
    (128, 256, 64), (2048, 1792, 1536), (300, 520, 200), (1, 8, 8), (129, 264, 72),
    (1000, 2048, 1536), (513, 1536, 8960 // 4), (4096, 512, 256),
]


def _ref(x, w, b=None):
    y = x.double() @ w.double().t()
    return y if b is None else y + b.double()


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("bias", [False, True])
@pytest.mark.parametrize("ctas", [0, 3])
def test_product_and_bias(M, N, K, bias, ctas):
    from ginfer_b200.ops import gemm_bf16, gemm_prefill
    g = torch.Generator(device="cpu").manual_seed(M * 7 + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    b = torch.randn(N, generator=g).to(DEV) if bias else None
    want = _ref(x, w, b)
    got = gemm_prefill.gemm(x, w, b, torch.bfloat16, ctas=ctas)
    assert got is not None
    gemm_bf16.check_errors()
    torch.testing.assert_close(got.double(), want, atol=2e-2, rtol=1e-2)
    got32 = gemm_prefill.gemm(x, w, b, torch.float32, ctas=ctas)
    gemm_bf16.check_errors()
    torch.testing.assert_close(got32.double(), want, atol=1e-3, rtol=1e-4)
    # a token's result depends neither on the other tokens nor on how many CTAs share the tiles
    alone = gemm_prefill.gemm(x[:1].contiguous(), w, b, torch.float32)
    assert torch.equal(alone, got32[:1])


@pytest.mark.parametrize("M,I,K", [(2048, 8960, 1536), (5, 224, 96), (300, 304, 80), (1111, 520, 256)])
@pytest.mark.parametrize("ctas", [0, 5])
def test_gated_epilogue(M, I, K, ctas):
    from ginfer_b200.ops import gemm_bf16, gemm_prefill
    g = torch.Generator(device="cpu").manual_seed(I)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    gate = (torch.randn(I, K, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    up = (torch.randn(I, K, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    inter = torch.stack([gate, up], dim=1).reshape(2 * I, K).contiguous()
    gg = _ref(x, gate).to(torch.bfloat16).double()      # gate and up are rounded as a product's
    uu = _ref(x, up).to(torch.bfloat16).double()        # output would be, then combined in fp32
    want = gg / (1 + torch.exp(-gg)) * uu
    got = gemm_prefill.gemm(x, inter, None, torch.bfloat16, epi=2, ctas=ctas)
    assert got is not None and got.shape == (M, I)
    gemm_bf16.check_errors()
    torch.testing.assert_close(got.double(), want, atol=2e-2, rtol=2e-2)


def test_shapes_it_does_not_take_are_handed_back():
    from ginfer_b200.ops import gemm_prefill
    x = torch.zeros(64, 60, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(32, 60, dtype=torch.bfloat16, device=DEV)
    assert gemm_prefill.gemm(x, w) is None                                  # K no multiple of 8
    x = torch.zeros(64, 64, dtype=torch.bfloat16, device=DEV)
    assert gemm_prefill.gemm(x, torch.zeros(36, 64, dtype=torch.bfloat16, device=DEV)) is None
    assert gemm_prefill.gemm(x, torch.zeros(40, 64, dtype=torch.bfloat16, device=DEV),
                             epi=2) is None                                 # pairs: N % 16
