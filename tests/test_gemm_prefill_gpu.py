"""The persistent tcgen05 product for many tokens alone against a float64 product of the same bf16
operands: tiles that are cut by M, N and K, more tiles than CTAs (both accumulators and every
ring stage are used again), bias, fp32 output, the gated epilogue; on single CTAs and on CTA pairs
(tiles of 256 tokens whose products read both CTAs' shared memory)."""
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
@pytest.mark.parametrize("pair", [False, True])
def test_product_and_bias(M, N, K, bias, ctas, pair):
    from ginfer_b200.ops import gemm_bf16, gemm_prefill
    g = torch.Generator(device="cpu").manual_seed(M * 7 + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    b = torch.randn(N, generator=g).to(DEV) if bias else None
    want = _ref(x, w, b)
    got = gemm_prefill.gemm(x, w, b, torch.bfloat16, ctas=ctas, pair=pair)
    assert got is not None
    gemm_bf16.check_errors()
    torch.testing.assert_close(got.double(), want, atol=2e-2, rtol=1e-2)
    got32 = gemm_prefill.gemm(x, w, b, torch.float32, ctas=ctas, pair=pair)
    gemm_bf16.check_errors()
    torch.testing.assert_close(got32.double(), want, atol=1e-3, rtol=1e-4)
    # a token's result depends neither on the other tokens nor on how many CTAs share the tiles
    alone = gemm_prefill.gemm(x[:1].contiguous(), w, b, torch.float32, pair=pair)
    assert torch.equal(alone, got32[:1])


@pytest.mark.parametrize("M,I,K", [(2048, 8960, 1536), (5, 224, 96), (300, 304, 80), (1111, 520, 256)])
@pytest.mark.parametrize("ctas", [0, 5])
@pytest.mark.parametrize("pair", [False, True])
def test_gated_epilogue(M, I, K, ctas, pair):
    from ginfer_b200.ops import gemm_bf16, gemm_prefill
    g = torch.Generator(device="cpu").manual_seed(I)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    gate = (torch.randn(I, K, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    up = (torch.randn(I, K, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    inter = torch.stack([gate, up], dim=1).reshape(2 * I, K).contiguous()
    gg = _ref(x, gate).to(torch.bfloat16).double()      # gate and up are rounded as a product's
    uu = _ref(x, up).to(torch.bfloat16).double()        # output would be, then combined in fp32
    want = gg / (1 + torch.exp(-gg)) * uu
    got = gemm_prefill.gemm(x, inter, None, torch.bfloat16, epi=2, ctas=ctas, pair=pair)
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


def _plain_qkv(x, w, b, table, positions, slots, nh, nkv, hd):
    """Bias, rounding to bf16, rotation in pairs (j, j + hd / 2), rounding: in float64 on the host."""
    qkv = _ref(x, w, b).to(torch.bfloat16).double().cpu()
    T = qkv.shape[0]
    cs = table.double().cpu()[positions.cpu().long()]            # [T, hd]: cos | sin
    cos, sin = cs[:, None, :hd // 2], cs[:, None, hd // 2:]
    heads = qkv.view(T, nh + 2 * nkv, hd).clone()
    lo, hi = heads[:, :nh + nkv, :hd // 2].clone(), heads[:, :nh + nkv, hd // 2:].clone()
    heads[:, :nh + nkv, :hd // 2] = lo * cos - hi * sin
    heads[:, :nh + nkv, hd // 2:] = lo * sin + hi * cos
    return heads.to(torch.bfloat16).double()


@pytest.mark.parametrize("M,K,nh,nkv,hd", [
    (2048, 1536, 12, 2, 128),      # the benchmark's layer
    (300, 200, 3, 1, 64),          # a tile cut by M, heads that do not fill a tile of 256 rows
    (129, 72, 5, 5, 64),           # 15 heads of 64: the last half tile holds one head
    (1100, 256, 4, 2, 128),
    (1, 64, 1, 1, 128),
])
@pytest.mark.parametrize("bias", [True, False])
@pytest.mark.parametrize("ctas", [0, 3])
def test_qkv_epilogue_rotates_and_writes_the_cache(M, K, nh, nkv, hd, bias, ctas):
    from ginfer_b200.ops import gemm_bf16, gemm_prefill, rope_kv_write
    g = torch.Generator(device="cpu").manual_seed(M + hd)
    N = (nh + 2 * nkv) * hd
    page, max_pos = 16, 4096
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    b = torch.randn(N, generator=g).to(DEV) if bias else None
    ang = torch.rand(max_pos, hd // 2, generator=g) * 6.283
    table = torch.cat([ang.cos(), ang.sin()], dim=1).float().contiguous().to(DEV)
    positions = torch.randint(0, max_pos, (M,), generator=g).int().to(DEV)
    npages = (M + page - 1) // page + 3
    slots = torch.randperm(npages * page, generator=g)[:M].int()      # every token a slot of its own
    if M > 4:
        slots[M // 2] = -1                                            # one token is not cached
    slots = slots.to(DEV)
    pages = torch.full((2, npages, page, nkv, hd), 7.0, dtype=torch.bfloat16, device=DEV)

    got = gemm_prefill.qkv_rope_write(x, w, b, table, hd, positions, slots, pages, nh, nkv, hd,
                                      min_tokens=1, ctas=ctas)
    assert got is not None and got.shape == (M, N)
    gemm_bf16.check_errors()

    want = _plain_qkv(x, w, b, table, positions, slots, nh, nkv, hd)   # [M, heads, hd]
    torch.testing.assert_close(got.double().cpu().view(M, -1, hd), want, atol=3e-2, rtol=2e-2)
    # the cache holds exactly what `out` holds for k and v, at the token's slot; nothing else moved
    flat = pages.view(2, npages * page, nkv, hd)
    keep = (slots >= 0).nonzero().flatten()
    idx = slots[keep].long()
    outh = got.view(M, nh + 2 * nkv, hd)
    assert torch.equal(flat[0][idx], outh[keep, nh:nh + nkv])
    assert torch.equal(flat[1][idx], outh[keep, nh + nkv:])
    untouched = torch.ones(npages * page, dtype=torch.bool, device=DEV)
    untouched[idx] = False
    assert (flat[:, untouched] == 7.0).all()

    # and it agrees with the plain product followed by the rotation kernel, which rotates q in
    # place and k on its way into the cache (its k columns of `qkv` stay as the product left them)
    qkv2 = gemm_prefill.gemm(x, w, b, torch.bfloat16)
    pages2 = torch.full_like(pages, 7.0)
    rope_kv_write(qkv2, table, hd, positions, slots, pages2, nh, nkv, hd)
    for cols in (slice(0, nh * hd), slice((nh + nkv) * hd, N)):
        torch.testing.assert_close(got[:, cols].float(), qkv2[:, cols].float(), atol=3e-2, rtol=2e-2)
    torch.testing.assert_close(pages.float(), pages2.float(), atol=3e-2, rtol=2e-2)


def test_qkv_epilogue_hands_back_what_it_does_not_take():
    from ginfer_b200.ops import gemm_prefill
    nh, nkv, hd, M, K = 2, 1, 48, 64, 64
    x = torch.zeros(M, K, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros((nh + 2 * nkv) * hd, K, dtype=torch.bfloat16, device=DEV)
    table = torch.zeros(8, hd, device=DEV)
    pos = torch.zeros(M, dtype=torch.int32, device=DEV)
    pages = torch.zeros(2, 8, 16, nkv, hd, dtype=torch.bfloat16, device=DEV)
    args = (pos, pos, pages, nh, nkv, hd)
    assert gemm_prefill.qkv_rope_write(x, w, None, table, hd, *args, min_tokens=1) is None  # hd 48
    nh, nkv, hd = 2, 1, 64
    w = torch.zeros((nh + 2 * nkv) * hd, K, dtype=torch.bfloat16, device=DEV)
    pages = torch.zeros(2, 8, 16, nkv, hd, dtype=torch.bfloat16, device=DEV)
    part = torch.zeros(8, 32, device=DEV)                                  # half the head rotated
    assert gemm_prefill.qkv_rope_write(x, w, None, part, 32, pos, pos, pages, nh, nkv, hd,
                                       min_tokens=1) is None
    assert gemm_prefill.qkv_rope_write(x, w, None, None, 0, pos, pos, pages, nh, nkv, hd,
                                       min_tokens=1) is None               # no rotation at all
