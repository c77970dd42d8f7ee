"""Each kernel alone against a plain PyTorch reference of the same operation, at sizes other than
the tiny models': widths and vocabularies that are no power of two, head sizes in steps of 16,
odd head counts and groups, page sizes, windows, and inputs made so that a fault shows."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _tol(dtype):
    return dict(atol=2e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H", [8, 100, 1536, 3])
def test_embedding(dtype, H):
    from ginfer_b200 import ops
    V = 777
    w = torch.randn(V, H, device=DEV).to(dtype)
    ids = torch.tensor([0, V - 1, 5, 5, 123, 776, 1], dtype=torch.int32, device=DEV)
    assert torch.equal(ops.embedding(ids, w), w[ids.long()])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,eps", [(96, 1e-5), (1536, 1e-6), (130, 1e-3), (5000, 1e-6),
                                   (13000, 1e-6)])
def test_add_rmsnorm(dtype, H, eps):
    from ginfer_b200 import ops
    T = 37
    x32 = torch.randn(T, H, device=DEV) * 3
    delta = (torch.randn(T, H, device=DEV)).to(dtype)
    for gdt in ({torch.float32, dtype}):
        gamma = (1 + 0.1 * torch.randn(H, device=DEV)).to(gdt)
        # residual in fp32 plus a delta in the activation type
        s, n = ops.add_rmsnorm(x32, delta, gamma, eps)
        want_s = x32.double() + delta.double()
        assert s.dtype == torch.float32
        torch.testing.assert_close(s.double(), want_s, atol=1e-6, rtol=1e-6)
        rms = torch.sqrt((want_s ** 2).sum(-1, keepdim=True) / H + eps)
        want_n = want_s * gamma.double() / rms
        torch.testing.assert_close(n.double(), want_n, **_tol(dtype))
        # no delta, activation-typed x (the embedding's output): s is x itself
        xa = x32.to(dtype)
        s2, n2 = ops.add_rmsnorm(xa, None, gamma, eps)
        assert s2 is xa
        xd = xa.double()
        want2 = xd * gamma.double() / torch.sqrt((xd ** 2).sum(-1, keepdim=True) / H + eps)
        torch.testing.assert_close(n2.double(), want2, **_tol(dtype))
        # selected rows only, no sum wanted (the final norm at the rows that want logits)
        rows = torch.tensor([36, 0, 7, 7], dtype=torch.int32, device=DEV)
        s3, n3 = ops.add_rmsnorm(x32, delta, gamma, eps, rows=rows, want_sum=False)
        assert s3 is None
        torch.testing.assert_close(n3.double(), want_n[rows.long()], **_tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,rot", [(4, 2, 16, 16), (3, 1, 32, 32), (5, 5, 48, 24),
                                           (12, 2, 128, 128), (2, 1, 64, 0)])
def test_rope_kv_write(dtype, nh, nkv, hd, rot):
    from ginfer_b200 import ops
    T, P, pages_n, maxpos = 19, 4, 11, 300
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device=DEV).to(dtype)
    orig = qkv.clone()
    positions = torch.randint(0, maxpos, (T,), device=DEV, dtype=torch.int32)
    slots = torch.randperm(pages_n * P, device=DEV)[:T].to(torch.int32)
    slots[3] = -1                                         # a token that is not to be written
    table = None
    if rot:
        half = rot // 2
        inv = 1.0 / (10000.0 ** (torch.arange(half, dtype=torch.float64) / half))
        ang = torch.arange(maxpos, dtype=torch.float64)[:, None] * inv[None, :]
        table = torch.cat([ang.cos(), ang.sin()], 1).float().to(DEV)
    pages = torch.full((2, pages_n, P, nkv, hd), 7.0, device=DEV).to(dtype)
    ops.rope_kv_write(qkv, table, rot, positions, slots, pages, nh, nkv, hd)

    def rotate(x):                                        # x [T, heads, hd], float64
        if not rot:
            return x
        half = rot // 2
        c = table[positions.long(), :half].double()[:, None, :]
        s = table[positions.long(), half:].double()[:, None, :]
        a, b = x[..., :half], x[..., half:rot]
        return torch.cat([a * c - b * s, a * s + b * c, x[..., rot:]], -1)
    o = orig.double()
    q_want = rotate(o[:, :nh * hd].reshape(T, nh, hd))
    k_want = rotate(o[:, nh * hd:(nh + nkv) * hd].reshape(T, nkv, hd))
    v_want = o[:, (nh + nkv) * hd:].reshape(T, nkv, hd)
    tol = _tol(dtype)
    torch.testing.assert_close(qkv[:, :nh * hd].double().reshape(T, nh, hd), q_want, **tol)
    assert torch.equal(qkv[:, (nh + nkv) * hd:], orig[:, (nh + nkv) * hd:])    # v untouched
    flatk = pages[0].reshape(pages_n * P, nkv, hd).double()
    flatv = pages[1].reshape(pages_n * P, nkv, hd).double()
    written = slots >= 0
    torch.testing.assert_close(flatk[slots[written].long()], k_want[written], **tol)
    torch.testing.assert_close(flatv[slots[written].long()], v_want[written], atol=0, rtol=0)
    untouched = torch.ones(pages_n * P, dtype=torch.bool, device=DEV)
    untouched[slots[written].long()] = False
    assert (flatk[untouched] == 7.0).all() and (flatv[untouched] == 7.0).all()
    # without a slot mapping nothing is written (a layer reading another layer's cache)
    pages2 = torch.full_like(pages, 7.0)
    ops.rope_kv_write(orig.clone(), table, rot, positions, None, pages2, nh, nkv, hd)
    assert (pages2 == 7.0).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_mul(dtype):
    from ginfer_b200 import ops
    T, I = 13, 1001
    gu = (torch.randn(T, 2 * I, device=DEV) * 4).to(dtype)
    g, u = gu[:, 0::2].double(), gu[:, 1::2].double()
    want = g / (1 + torch.exp(-g)) * u
    torch.testing.assert_close(ops.silu_mul(gu).double(), want, **_tol(dtype))


@pytest.mark.parametrize("M,N,K", [(2, 8, 9), (1, 389, 96), (130, 2000, 408), (64, 64, 16),
                                   (257, 1001, 1000), (7, 3, 5)])
@pytest.mark.parametrize("bias", [False, True])
def test_gemm_f32_is_true_fp32(M, N, K, bias):
    from ginfer_b200.ops.linear import gemm_f32
    # values with 20 significant bits: a tf32 or bf16 product would lose them
    x = (torch.randn(M, K, device=DEV) * 1024).round() / 1024 + 1.0
    w = (torch.randn(N, K, device=DEV) * 1024).round() / 1024
    b = torch.randn(N, device=DEV) if bias else None
    got = gemm_f32(x, w, b)
    want = x.double() @ w.double().t() + (b.double() if bias else 0)
    torch.testing.assert_close(got.double(), want, atol=2e-5 * math.sqrt(K), rtol=2e-6)
    # a row's result does not depend on the other rows of the batch
    assert torch.equal(gemm_f32(x[:1].contiguous(), w, b), got[:1])


def _paged_case(B_lens, q_lens, nh, nkv, hd, P, window, dtype, seed=0, spike=True):
    """Random paged cache and queries for requests with kv lengths ``B_lens`` whose last
    ``q_lens`` tokens are this step's queries.  Returns the kernel inputs and the plain result."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    B = len(B_lens)
    total_pages = sum(-(-n // P) for n in B_lens) + 5
    perm = torch.randperm(total_pages, generator=g).tolist()
    W = max(-(-n // P) for n in B_lens) + 2
    table = torch.full((B, W), -1, dtype=torch.int32)
    pages = torch.zeros(2, total_pages, P, nkv, hd)
    ks, vs, qs = [], [], []
    at = 0
    for b, n in enumerate(B_lens):
        k = torch.randn(n, nkv, hd, generator=g)
        v = torch.randn(n, nkv, hd, generator=g)
        q = torch.randn(q_lens[b], nh, hd, generator=g)
        if spike and n > 40:
            # one far key stands out for one query: scale them so that its score dominates
            far = 3 if window <= 0 else max(0, n - min(window, n))   # the oldest visible key
            q[-1, 0] = 0
            q[-1, 0, 0] = 30.0
            k[far, 0] = 0
            k[far, 0, 0] = 30.0
        ks.append(k), vs.append(v), qs.append(q)
        for i in range(-(-n // P)):
            page = perm[at]
            at += 1
            table[b, i] = page
            m = min(P, n - i * P)
            pages[0, page, :m] = k[i * P:i * P + m]
            pages[1, page, :m] = v[i * P:i * P + m]
    pages = pages.to(dtype)
    qcat = torch.cat(qs).to(dtype)
    scale = 1.0 / math.sqrt(hd)
    want = []
    for b, n in enumerate(B_lens):
        k = pages[0].double().reshape(-1, nkv, hd)
        v = pages[1].double().reshape(-1, nkv, hd)
        idx = torch.tensor([table[b, c // P] * P + c % P for c in range(n)])
        kk, vv = k[idx], v[idx]
        q = qs[b].to(dtype).double()
        ql = q_lens[b]
        out = torch.empty(ql, nh, hd, dtype=torch.float64)
        for r in range(ql):
            p = n - ql + r
            lo = max(0, p - window + 1) if window > 0 else 0
            for h in range(nh):
                kvh = h // (nh // nkv)
                s = (kk[lo:p + 1, kvh] @ q[r, h]) * scale
                out[r, h] = torch.softmax(s, 0) @ vv[lo:p + 1, kvh]
        want.append(out)
    want = torch.cat(want).reshape(-1, nh * hd)
    # windowed layers have given back the pages no query of this step can see
    if window > 0:
        for b, n in enumerate(B_lens):
            first_visible = max(0, n - q_lens[b] - window + 1)
            table[b, :first_visible // P] = -1
    cu = [0]
    for ql in q_lens:
        cu.append(cu[-1] + ql)
    positions = torch.cat([torch.arange(n - ql, n) for n, ql in zip(B_lens, q_lens)])
    seq_of_token = torch.cat([torch.full((ql,), b) for b, ql in enumerate(q_lens)])
    dev = dict(
        q=qcat.reshape(-1, nh * hd).to(DEV), pages=pages.to(DEV), table=table.to(DEV),
        cu=torch.tensor(cu, dtype=torch.int32, device=DEV),
        kv_lens=torch.tensor(B_lens, dtype=torch.int32, device=DEV),
        positions=positions.to(torch.int32).to(DEV),
        seq_of_token=seq_of_token.to(torch.int32).to(DEV))
    return dev, want, scale


def _qkv(dev, nh, nkv, hd):
    """Queries as the first columns of a wider row, as the engine's joined projection has them."""
    T = dev["q"].shape[0]
    qkv = torch.full((T, (nh + 2 * nkv) * hd), float("nan"), dtype=dev["q"].dtype, device=DEV)
    qkv[:, :nh * hd] = dev["q"]
    return qkv


ATT_CASES = [
    # kv lens, q lens, nh, nkv, hd, page, window
    ([70, 5, 130], [70, 5, 130], 4, 2, 16, 16, 0),
    ([200, 64, 1], [3, 64, 1], 3, 1, 32, 8, 0),
    ([300, 129, 77], [100, 1, 77], 5, 5, 48, 4, 33),
    ([515, 260], [2, 260], 12, 2, 128, 16, 0),
    ([700, 90], [65, 90], 6, 3, 64, 16, 100),
    ([1100], [1100], 14, 2, 64, 32, 0),
    # head sizes that are no multiples of 32 or 64, and one of three 64-channel parts
    ([130, 40, 260], [130, 1, 37], 4, 2, 80, 16, 0),
    ([200, 33], [64, 33], 2, 1, 112, 8, 20),
    ([300, 70], [5, 70], 6, 2, 192, 16, 50),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", ATT_CASES)
def test_paged_attention_simt(dtype, case):
    from ginfer_b200 import ops
    lens, qls, nh, nkv, hd, P, window = case
    dev, want, scale = _paged_case(lens, qls, nh, nkv, hd, P, window, dtype)
    out = ops.paged_attention_simt(_qkv(dev, nh, nkv, hd), dev["pages"], dev["table"],
                                   dev["seq_of_token"], dev["positions"], nh, nkv, hd, scale,
                                   window, P)
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=1e-2, rtol=2e-2)
    torch.testing.assert_close(out.double().cpu(), want, **tol)


@pytest.mark.parametrize("case", ATT_CASES)
def test_attention_bf16_prefill(case):
    from ginfer_b200.ops import attention_bf16
    lens, qls, nh, nkv, hd, P, window = case
    dev, want, scale = _paged_case(lens, qls, nh, nkv, hd, P, window, torch.bfloat16)
    out = attention_bf16.prefill(_qkv(dev, nh, nkv, hd), dev["pages"], dev["table"], dev["cu"],
                                 dev["kv_lens"], len(lens), max(qls), nh, nkv, hd, scale, window,
                                 P)
    torch.testing.assert_close(out.double().cpu(), want, atol=1e-2, rtol=2e-2)


TC_CASES = [
    # kv lens, q lens, nh, nkv, hd, page, window
    ([515, 260], [2, 260], 12, 2, 128, 16, 0),
    ([700, 90], [65, 90], 6, 3, 64, 16, 100),
    ([1100], [1100], 14, 2, 64, 32, 0),
    ([300, 129, 77, 1000], [300, 1, 77, 129], 4, 4, 128, 8, 0),
    ([640, 400], [128, 400], 2, 1, 128, 16, 200),
    ([2048], [2048], 4, 2, 128, 16, 0),
    # many key tiles per query tile: pairs of CTAs share them (also with a window, and where the
    # second CTA's keys are all behind the window's start for the first rows)
    ([1800, 900], [700, 900], 6, 2, 128, 16, 700),
    ([3000], [130], 4, 1, 64, 8, 0),
]


@pytest.mark.parametrize("case", TC_CASES)
def test_attention_tcgen05_prefill(case):
    from ginfer_b200.ops import attention_bf16, gemm_bf16
    lens, qls, nh, nkv, hd, P, window = case
    dev, want, scale = _paged_case(lens, qls, nh, nkv, hd, P, window, torch.bfloat16)
    out = attention_bf16.prefill_tc(_qkv(dev, nh, nkv, hd), dev["pages"], dev["table"], dev["cu"],
                                    dev["kv_lens"], len(lens), max(qls), nh, nkv, hd, scale,
                                    window, P)
    assert out is not None
    gemm_bf16.check_errors()
    torch.testing.assert_close(out.double().cpu(), want, atol=1e-2, rtol=2e-2)


@pytest.mark.parametrize("case", [TC_CASES[1], TC_CASES[5], TC_CASES[6]])
@pytest.mark.parametrize("every", [4, 2])
def test_attention_tcgen05_prefill_with_a_share_of_exponentials_by_polynomial(case, every):
    """The build that computes every n-th exponential of an unmasked tile by a cubic on the FMA
    pipe (off by default) against the oracle and against the default build."""
    from ginfer_b200.ops import attention_bf16, gemm_bf16
    lens, qls, nh, nkv, hd, P, window = case
    dev, want, scale = _paged_case(lens, qls, nh, nkv, hd, P, window, torch.bfloat16)
    args = (_qkv(dev, nh, nkv, hd), dev["pages"], dev["table"], dev["cu"], dev["kv_lens"],
            len(lens), max(qls), nh, nkv, hd, scale, window, P)
    out = attention_bf16.prefill_tc(*args, poly_exp_every=every)
    assert out is not None
    gemm_bf16.check_errors()
    torch.testing.assert_close(out.double().cpu(), want, atol=1e-2, rtol=2e-2)
    plain = attention_bf16.prefill_tc(*args, poly_exp_every=0)
    torch.testing.assert_close(out.float(), plain.float(), atol=1e-2, rtol=2e-2)


DEC_CASES = [
    ([70, 5, 130, 1], 4, 2, 16, 16, 0),
    ([200, 64, 1, 63, 65], 3, 1, 32, 8, 0),
    ([300, 129, 77], 5, 5, 48, 4, 33),
    ([515, 260, 4000], 12, 2, 128, 16, 0),
    ([700, 90], 6, 3, 64, 16, 100),
    ([2049, 17], 40, 2, 64, 16, 0),               # 20 query heads per kv head: two chunks of 16
    ([130, 40, 700], 6, 2, 80, 16, 0),            # five steps of 16 channels
    ([300, 70], 6, 2, 192, 8, 50),
]


@pytest.mark.parametrize("case", DEC_CASES)
@pytest.mark.parametrize("splits", [1, 2, 5, 8, 16, -4])
def test_attention_bf16_decode(case, splits):
    from ginfer_b200.ops import attention_bf16
    lens, nh, nkv, hd, P, window = case
    qls = [1] * len(lens)
    dev, want, scale = _paged_case(lens, qls, nh, nkv, hd, P, window, torch.bfloat16)
    # 2, 4, 8, 16 merge inside a cluster; other counts (and negative ones here) through scratch
    out = attention_bf16.decode(_qkv(dev, nh, nkv, hd), dev["pages"], dev["table"], dev["cu"],
                                dev["positions"], len(lens), nh, nkv, hd, scale, window, P,
                                abs(splits), through_scratch=splits < 0)
    torch.testing.assert_close(out.double().cpu(), want, atol=1e-2, rtol=2e-2)


DEC_TMA_CASES = [   # what the kernel that loads by TMA serves: page sizes and head sizes
    ([300, 64, 1, 65, 129], 8, 1, 128, 8, 0),
    ([1000, 130, 63], 14, 2, 64, 32, 0),
    ([700, 257, 64], 16, 2, 128, 64, 300),
    ([900, 5], 4, 4, 256, 128, 0),
    ([1500, 700], 6, 3, 128, 16, 130),           # a window that starts inside a tile
    ([4100], 18, 2, 64, 16, 0),                   # 9 query heads per kv head: two chunks of 8
    ([300, 70, 8], 4, 2, 256, 8, 0),              # 64 boxes a tile: two for each lane of the loader
    ([600, 70, 9], 6, 2, 192, 16, 40),            # three 64-channel parts a row
]


@pytest.mark.parametrize("case", DEC_TMA_CASES)
@pytest.mark.parametrize("splits", [1, 2, 4, 8, 16])
def test_attention_bf16_decode_with_tiles_by_tma(case, splits):
    """The decode kernel that loads by TMA against the oracle and against the kernel that gathers
    with 16-byte copies (the same arithmetic in another tile layout: equal within rounding)."""
    from ginfer_b200.ops import attention_bf16, gemm_bf16
    lens, nh, nkv, hd, P, window = case
    dev, want, scale = _paged_case(lens, [1] * len(lens), nh, nkv, hd, P, window, torch.bfloat16)
    args = (_qkv(dev, nh, nkv, hd), dev["pages"], dev["table"], dev["cu"], dev["positions"],
            len(lens), nh, nkv, hd, scale, window, P, splits)
    assert attention_bf16.tma_serves(hd, P, splits)
    out = attention_bf16.decode(*args)
    gemm_bf16.check_errors()
    torch.testing.assert_close(out.double().cpu(), want, atol=1e-2, rtol=2e-2)
    other = attention_bf16.decode(*args, use_tma=False)
    torch.testing.assert_close(out.float(), other.float(), atol=1e-2, rtol=2e-2)


@pytest.mark.parametrize("case", [DEC_TMA_CASES[0], DEC_TMA_CASES[2], DEC_TMA_CASES[4],
                                  DEC_TMA_CASES[5], ([9000, 300, 2100], 12, 2, 128, 16, 0)])
@pytest.mark.parametrize("splits,parts", [(8, 2), (8, 5), (4, 3), (1, 4), (8, 16)])
def test_attention_bf16_decode_with_several_clusters_a_request(case, splits, parts):
    """Few requests with many keys: several clusters share a request's keys and a second kernel
    adds their results up.  Against the oracle and against one cluster a request; parts that get
    no key at all (more pieces than tiles) count for nothing."""
    from ginfer_b200.ops import attention_bf16, gemm_bf16
    lens, nh, nkv, hd, P, window = case
    dev, want, scale = _paged_case(lens, [1] * len(lens), nh, nkv, hd, P, window, torch.bfloat16)
    args = (_qkv(dev, nh, nkv, hd), dev["pages"], dev["table"], dev["cu"], dev["positions"],
            len(lens), nh, nkv, hd, scale, window, P, splits)
    out = attention_bf16.decode(*args, parts=parts)
    gemm_bf16.check_errors()
    torch.testing.assert_close(out.double().cpu(), want, atol=1e-2, rtol=2e-2)
    one = attention_bf16.decode(*args)
    torch.testing.assert_close(out.float(), one.float(), atol=1e-2, rtol=2e-2)


@pytest.mark.parametrize("case", DEC_CASES)
@pytest.mark.parametrize("splits", [1, 4, 8, -3])
@pytest.mark.parametrize("rot_frac", [1.0, 0.5])
def test_attention_bf16_decode_rotates_and_writes_the_cache_itself(case, splits, rot_frac):
    """The decode kernel given unrotated q and k equals the rotation-and-write kernel followed by
    the decode kernel, bit for bit in the cache and in the output."""
    from ginfer_b200 import ops
    from ginfer_b200.ops import attention_bf16
    lens, nh, nkv, hd, P, window = case
    B = len(lens)
    dev, _, scale = _paged_case(lens, [1] * B, nh, nkv, hd, P, window, torch.bfloat16, spike=False)
    g = torch.Generator().manual_seed(5)
    qkv = torch.randn(B, (nh + 2 * nkv) * hd, generator=g).to(torch.bfloat16).cuda()
    rot = int(hd * rot_frac) // 2 * 2
    ang = torch.rand(max(lens) + 1, rot // 2, generator=g) * 6.28
    table = torch.cat([ang.cos(), ang.sin()], dim=1).float().cuda().contiguous()
    slots = torch.tensor([int(dev["table"][b, (n - 1) // P]) * P + (n - 1) % P
                          for b, n in enumerate(lens)], dtype=torch.int32).cuda()
    # separately: rotate q in place, write k and v, then attend
    qkv_a, pages_a = qkv.clone(), dev["pages"].clone()
    ops.rope_kv_write(qkv_a, table, rot, dev["positions"], slots, pages_a, nh, nkv, hd)
    want = attention_bf16.decode(qkv_a, pages_a, dev["table"], dev["cu"], dev["positions"], B, nh,
                                 nkv, hd, scale, window, P, abs(splits),
                                 through_scratch=splits < 0)
    # in one kernel
    pages_b = dev["pages"].clone()
    got = attention_bf16.decode(qkv.clone(), pages_b, dev["table"], dev["cu"], dev["positions"],
                                B, nh, nkv, hd, scale, window, P, abs(splits),
                                through_scratch=splits < 0, rope=(table, rot, True))
    torch.cuda.synchronize()
    assert torch.equal(pages_b, pages_a), "the cache differs"
    assert torch.equal(got, want)
    # without the write, the cache stays as it was
    pages_c = dev["pages"].clone()
    attention_bf16.decode(qkv.clone(), pages_c, dev["table"], dev["cu"], dev["positions"], B, nh,
                          nkv, hd, scale, window, P, abs(splits), through_scratch=splits < 0,
                          rope=(table, rot, False))
    torch.cuda.synchronize()
    assert torch.equal(pages_c, dev["pages"])


def test_attention_refuses_head_sizes_it_cannot_take():
    from ginfer_b200 import ops
    from ginfer_b200.ops import attention_bf16
    assert not attention_bf16.supports(40, 4, 2) and not attention_bf16.supports(272, 4, 2)
    assert attention_bf16.supports(48, 5, 5) and attention_bf16.supports(256, 8, 1)
    dev, _, scale = _paged_case([20], [20], 2, 1, 16, 16, 0, torch.float32, spike=False)
    q = torch.zeros(20, 2 * 272 * 2, device=DEV)
    with pytest.raises(ValueError, match="head sizes up to 256"):
        ops.paged_attention_simt(q, torch.zeros(2, 4, 16, 1, 272, device=DEV), dev["table"],
                                 dev["seq_of_token"], dev["positions"], 2, 1, 272, scale, 0, 16)


@pytest.mark.parametrize("V", [256, 389, 151936, 7])
def test_argmax_lowest_index_wins(V):
    from ginfer_b200 import ops
    x = torch.randn(6, V, device=DEV)
    x[1, V - 1] = 50.0
    x[2, 0] = 50.0
    x[3, [V // 2, V // 3, V - 1]] = 60.0                  # a tie: the lowest index wins
    x[4] = -3.0                                           # all equal: index 0
    x[5, 1] = float("nan")                                # NaN never wins
    got = ops.argmax(x).tolist()
    want = [int(x[0].argmax()), V - 1, 0, V // 3, 0,
            int(torch.where(torch.isnan(x[5]), torch.tensor(-1e30, device=DEV), x[5]).argmax())]
    assert got == want


@pytest.mark.parametrize("V", [389, 5000, 151936])
def test_temperature_sampling_is_the_inverse_cdf(V):
    from ginfer_b200 import ops
    R = 64
    g = torch.Generator(device="cpu").manual_seed(V)
    logits = (torch.randn(R, V, generator=g) * 3).to(DEV)
    temps = torch.full((R,), 0.8, device=DEV)
    temps[0] = 0.0                                        # greedy row inside a sampled batch
    temps[1] = 1e-3                                       # nearly greedy
    u = torch.rand(R, generator=g).to(DEV)
    u[2], u[3] = 0.0, 0.99999994
    got = ops.sample(logits, temps, u).tolist()
    assert got[0] == int(logits[0].argmax()) and got[1] == int(logits[1].argmax())
    for r in range(2, R):
        p = torch.softmax(logits[r].double() / float(temps[r]), -1)
        cdf = torch.cumsum(p, 0)
        want = min(int(torch.searchsorted(cdf, u[r].double())), V - 1)
        if got[r] != want:                                # u within rounding of a CDF step
            lo, hi = sorted((got[r], want))
            assert float(cdf[hi - 1] - cdf[lo]).__abs__() < 1e-5 or \
                abs(float(cdf[lo]) - float(u[r])) < 1e-5, (r, got[r], want)
    # the distribution: many draws of one row follow softmax
    row = torch.tensor([[2.0, 1.0, 0.0, -1.0, 0.5]], device=DEV).repeat(4000, 1)
    us = torch.rand(4000, generator=g).to(DEV)
    picks = ops.sample(row, torch.full((4000,), 0.7, device=DEV), us)
    freq = torch.bincount(picks.long(), minlength=5).double() / 4000
    want = torch.softmax(row[0].double() / 0.7, -1).cpu()
    assert (freq.cpu() - want).abs().max() < 0.03
