"""bf16 matrix products on the 5th-generation tensor cores (``csrc/gemm_bf16.cu``: tcgen05.mma with
the accumulator in tensor memory, operands staged by TMA)."""
from __future__ import annotations

from ctypes import c_int, c_void_p

import torch

NUM_SMS = 148
_state: dict = {}


def _dev_state(device):
    key = device.index if device.index is not None else torch.cuda.current_device()
    st = _state.get(key)
    if st is None:
        st = {"err": torch.zeros(1, dtype=torch.int32, device=device), "ws": None}
        _state[key] = st
    return st


def check_errors(device="cuda:0") -> None:
    """Raise if a kernel gave up a bounded wait since the last check (reads one int back)."""
    st = _state.get(torch.device(device).index or 0)
    if st is None:
        return
    code = int(st["err"].item())
    if code:
        st["err"].zero_()
        raise RuntimeError(f"gemm_bf16: a wait inside the tcgen05 kernel ran out (role {code}: "
                           "1 = TMA producer, 2 = MMA issuer, 3 = epilogue)")


def error_word(device="cuda:0") -> torch.Tensor:
    """The device int that kernels set when a bounded wait runs out (for a caller that reads it
    back together with other results instead of calling :func:`check_errors`)."""
    return _dev_state(torch.device(device))["err"]


def raise_for(code: int, device="cuda:0") -> None:
    if code:
        _dev_state(torch.device(device))["err"].zero_()
        raise RuntimeError(f"gemm_bf16: a wait inside the tcgen05 kernel ran out (role {code}: "
                           "1 = TMA producer, 2 = MMA issuer, 3 = epilogue)")


def token_tile(M: int) -> int:
    return 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128 if M <= 128 else 256


def split_k_for(M: int, N: int, K: int) -> int:
    """Split the K range of products whose tiles alone would leave most SMs idle: 2, 4, 8 or 12
    splits, which form a thread-block cluster and add up through distributed shared memory."""
    tiles = -(-N // 128) * -(-M // token_tile(M))
    nkb = -(-K // 64)
    split = 1
    while split < 8 and tiles * split * 2 <= NUM_SMS + NUM_SMS // 4 and nkb // (split * 2) >= 2:
        split *= 2
    if split == 8 and tiles * 12 <= NUM_SMS and nkb // 12 >= 8:
        split = 12      # a long reduction on few tiles (the down product): 144 CTAs instead of 96
    if split == 1 and M <= 16 and NUM_SMS // 2 < tiles <= NUM_SMS and nkb >= 16:
        split = 2       # about one tile an SM (gate/up): pairs of CTAs have more under way
    return split


def _workspace(words: int, device) -> torch.Tensor:
    if torch.cuda.is_current_stream_capturing():
        return torch.empty(words, dtype=torch.float32, device=device)
    st = _dev_state(device)
    if st["ws"] is None or st["ws"].numel() < words:
        st["ws"] = torch.empty(max(words, 1 << 22), dtype=torch.float32, device=device)
    return st["ws"]


def supports(x: torch.Tensor, weight: torch.Tensor) -> bool:
    K = weight.shape[1]
    return (K % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def gemm(x, weight, bias_f32=None, out_dtype=torch.bfloat16, epi: int = 0, split_k=None,
         through_workspace: bool = False):
    """``x [M, K] @ weight[N, K]^T``; ``epi`` 0: (+ bias) -> ``[M, N]``; ``epi`` 2: weight rows
    are interleaved (gate_i, up_i) and the result is ``silu(gate) * up`` -> ``[M, N / 2]``.
    ``split_k``: None picks it; 2, 4 or 8 add up inside a cluster; with ``through_workspace`` any
    number of splits adds up through global memory.  Returns ``None`` if the kernel cannot serve
    the shape."""
    from . import _fn, _ok, _p, _stream
    if not supports(x, weight):
        return None
    M, K = x.shape
    N = weight.shape[0]
    cols = N // 2 if epi == 2 else N
    out = torch.empty((M, cols), dtype=out_dtype, device=x.device)
    if M == 0:
        return out
    sk = split_k_for(M, N, K) if split_k is None else int(split_k)
    ws = None
    if sk > 1 and through_workspace:
        bn = token_tile(M)
        ws = _workspace(-(-N // 128) * -(-M // bn) * sk * 128 * bn, x.device)
    st = _dev_state(x.device)
    f = _fn("gemm_bf16", "gf_gemm_bf16_tc",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
             c_int, c_int, c_void_p, c_void_p, c_void_p])
    rc = f(_p(x), x.stride(0), _p(weight), _p(bias_f32), _p(out), cols, M, N, K, int(epi),
           1 if out_dtype == torch.float32 else 0, sk, _p(ws), _p(st["err"]), _stream())
    if rc in (-6, -7):
        return None
    _ok(rc, "gemm_bf16_tc")
    return out


# The largest token count the gated product runs here for.  In a CUDA graph, 1.5B shapes, weights
# from HBM: 8 tokens 11.5 us (two K splits) against 12.6 for cuBLAS + SiLU*mul, 16 tokens 11.8
# against 12.6, 32 tokens 13.3 against 12.7, 64 tokens 14.8 against 13.7: every CTA streams the whole
# activation matrix beside its weights, which costs as much as the weights from 32 tokens on.
MAX_TOKENS = 16


def try_linear(x, weight, bias_f32, out_dtype):
    """Run the tcgen05 kernel where it is the faster one (the small batches of decode steps and
    short prompt portions); ``None`` hands the product to cuBLAS."""
    limit = PLAIN_MAX_TOKENS_LONG_K if weight.shape[1] >= LONG_K else PLAIN_MAX_TOKENS
    if x.shape[0] > limit:
        return None
    return gemm(x, weight, bias_f32, out_dtype, epi=0)


# Plain products leave for cuBLAS above this many tokens.  In a CUDA graph on a B200, 1.5B shapes,
# weights from HBM (us, here / cuBLAS): q/k/v 8 tokens 4.2 / 5.6, 16 tokens 4.6 / 4.6, 32 tokens
# 6.3 / 4.6; output 4.3 / 5.0, 4.7 / 4.6, 6.5 / 4.5; down (a reduction of 8,960) 8 tokens 8.6 / 16.9,
# 32 tokens 10.5 / 13.2, 48 tokens 12.6 / 13.2, 64 tokens 14.1 / 13.3.  With these limits the decode
# step at batch 32 and 64 is 8 % faster than with 32 tokens for all.
PLAIN_MAX_TOKENS = 16
PLAIN_MAX_TOKENS_LONG_K = 48   # for reductions of at least LONG_K
LONG_K = 4096


# ----------------------------------------------------------------------------- fused with the norm
FUSED_MAX_TOKENS = 32          # the fused kernels take token tiles of 16 and 32
SS_LD = 32                     # tokens per row of the partial sums of squares


def _cluster_split(N: int, K: int, k_share_max: int | None = None) -> int:
    """2, 4 or 8 K-splits (a thread-block cluster) for products whose row tiles alone would leave
    most SMs idle; ``k_share_max`` bounds the K range of one split (elements)."""
    tiles = -(-N // 128)
    nkb = -(-K // 64)
    split = 1
    while split < 8 and tiles * split * 2 <= NUM_SMS + NUM_SMS // 4 and nkb // (split * 2) >= 2:
        split *= 2
    while k_share_max is not None and split < 8 and -(-nkb // split) * 64 > k_share_max:
        split *= 2
    return split


def gemm_resid(x, weight, bias_f32, resid):
    """``s = resid + x @ weight^T (+ bias)`` in fp32 with, per token, the partial sums of
    ``s^2`` (``csrc/gemm_fused_norm.cu``).  Returns ``(s [M, N] fp32, sumsq [parts, 32] fp32)``
    or ``None`` if the kernel cannot serve the shapes."""
    from . import _fn, _ok, _p, _stream
    M, K = x.shape
    N = weight.shape[0]
    if M > FUSED_MAX_TOKENS or not supports(x, weight) or resid.dtype != torch.float32:
        return None
    if resid.shape != (M, N) or not resid.is_contiguous():
        return None
    split = _cluster_split(N, K)
    parts = -(-N // 128) * split
    out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    sumsq = torch.empty((parts, SS_LD), dtype=torch.float32, device=x.device)
    f = _fn("gemm_fused_norm", "gf_gemm_resid",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
             c_int, c_int, c_int, c_void_p, c_void_p])
    rc = f(_p(x), x.stride(0), _p(weight), _p(bias_f32), _p(resid), _p(out), _p(sumsq), SS_LD, M,
           N, K, split, _p(_dev_state(x.device)["err"]), _stream())
    if rc == -6:
        return None
    _ok(rc, "gemm_resid")
    return out, sumsq


def gemm_normed(resid, sumsq, gamma, eps, weight, bias_f32=None, out_dtype=torch.bfloat16,
                gated: bool = False):
    """``norm(resid) @ weight^T (+ bias)`` (or ``silu(gate) * up`` over row-interleaved weights)
    where ``norm`` is the RMS normalisation with ``gamma`` and the statistics a
    :func:`gemm_resid` left in ``sumsq``.  ``None`` if the kernel cannot serve the shapes."""
    from ctypes import c_float

    from . import _fn, _ok, _p, _stream
    M, K = resid.shape
    N = weight.shape[0]
    if M > FUSED_MAX_TOKENS or K % 8 or resid.dtype != torch.float32 or not resid.is_contiguous():
        return None
    if weight.data_ptr() % 16 or gamma.data_ptr() % 16 or gamma.numel() != K:
        return None
    bn = 16 if M <= 16 else 32
    # the CTA's share of the normalised operand stays in shared memory: at most 64 KB of it
    split = _cluster_split(N, K, k_share_max=(64 << 10) // (bn * 2))
    if -(-(-(-K // 64)) // split) * 64 * bn * 2 > (64 << 10):
        return None
    cols = N // 2 if gated else N
    out = torch.empty((M, cols), dtype=out_dtype, device=resid.device)
    f = _fn("gemm_fused_norm", "gf_gemm_normed",
            [c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_float, c_void_p, c_void_p,
             c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    rc = f(_p(resid), _p(sumsq), sumsq.shape[0], sumsq.stride(0), _p(gamma),
           1 if gamma.dtype == torch.float32 else 0, float(eps), _p(weight), _p(bias_f32), _p(out),
           cols, M, N, K, 1 if gated else 0, 1 if out_dtype == torch.float32 else 0, split,
           _p(_dev_state(resid.device)["err"]), _stream())
    if rc == -6:
        return None
    _ok(rc, "gemm_normed")
    return out
