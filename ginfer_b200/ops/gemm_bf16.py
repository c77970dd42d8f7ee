"""bf16 matrix products on the 5th-generation tensor cores (``csrc/gemm_bf16.cu``: tcgen05.mma with
the accumulator in tensor memory, operands staged by TMA)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_void_p
from dataclasses import dataclass

import torch

B200_SMS = 148                 # what the split choices assume where no device can be asked
_state: dict = {}
_sms: dict = {}


def num_sms(device=None) -> int:
    """Streaming multiprocessors of ``device`` (the current one if ``None``), read from the
    device; without a CUDA device (host-side tests of the split choices) a B200's count."""
    if not torch.cuda.is_available():
        return B200_SMS
    key = torch.device(device).index if device is not None else None
    if key is None:
        key = torch.cuda.current_device()
    n = _sms.get(key)
    if n is None:
        n = _sms[key] = torch.cuda.get_device_properties(key).multi_processor_count
    return n


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


def split_k_for(M: int, N: int, K: int, sms: int | None = None) -> int:
    """Split the K range of products whose tiles alone would leave most SMs idle: 2, 4, 8 or 12
    splits, which form a thread-block cluster and add up through distributed shared memory.
    ``sms``: the device's SM count (asked of the current device if ``None``)."""
    sms = sms or num_sms()
    tiles = -(-N // 128) * -(-M // token_tile(M))
    nkb = -(-K // 64)
    split = 1
    while split < 8 and tiles * split * 2 <= sms + sms // 4 and nkb // (split * 2) >= 2:
        split *= 2
    if split == 8 and tiles * 12 <= sms and nkb // 12 >= 8:
        split = 12      # a long reduction on few tiles (the down product): 144 CTAs instead of 96
    if split == 1 and M <= 64 and sms // 2 < tiles <= sms and nkb >= 16:
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


@dataclass
class RowScale:
    """Partial sums of squares ``sumsq [parts, ld]`` of the rows of a tensor of ``width`` columns
    with the ``eps`` of an RMS normalisation: a product whose operand is that tensor times gamma
    multiplies its accumulator by ``rsqrt(sum of the partials / width + eps)`` per token."""
    sumsq: torch.Tensor
    eps: float


def sumsq_ld(M: int) -> int:
    return -(-M // 16) * 16


def gemm(x, weight, bias_f32=None, out_dtype=torch.bfloat16, epi: int = 0, split_k=None,
         through_workspace: bool = False, scale: RowScale | None = None, resid=None, gamma=None):
    """``x [M, K] @ weight[N, K]^T``; ``epi`` 0: (+ bias) -> ``[M, N]``; ``epi`` 2: weight rows
    are interleaved (gate_i, up_i) and the result is ``silu(gate) * up`` -> ``[M, N / 2]``.
    ``split_k``: None picks it; 2, 4, 8 or 12 add up inside a cluster; with ``through_workspace``
    any number of splits adds up through global memory.  ``scale``: the accumulator of every token
    is multiplied by its factor first (a deferred RMS normalisation).  ``resid`` (fp32 ``[M, N]``): the result
    is ``(s, scaled, sumsq)`` with ``s = resid + x W^T (+ bias)`` in fp32, ``scaled = bf16(s *
    gamma)`` (``None`` without ``gamma``) and the partial sums of squares of ``s``'s rows.
    Returns ``None`` if the kernel cannot serve the shape."""
    from . import _fn, _ok, _p, _stream
    if not supports(x, weight):
        return None
    M, K = x.shape
    N = weight.shape[0]
    if resid is not None:
        if (M > RESID_MAX_TOKENS or through_workspace or resid.dtype != torch.float32
                or resid.shape != (M, N) or not resid.is_contiguous() or epi != 0):
            return None
        epi, out_dtype = 3, torch.float32
    cols = N // 2 if epi == 2 else N
    out = torch.empty((M, cols), dtype=out_dtype, device=x.device)
    if M == 0:
        return out if resid is None else None
    sk = split_k_for(M, N, K) if split_k is None else int(split_k)
    ws = None
    if sk > 1 and through_workspace:
        bn = token_tile(M)
        ws = _workspace(-(-N // 128) * -(-M // bn) * sk * 128 * bn, x.device)
    ld = sumsq_ld(M)
    in_sumsq, in_parts, in_eps = None, 0, 0.0
    if scale is not None:
        if scale.sumsq.stride(0) != ld or scale.sumsq.dtype != torch.float32:
            return None
        in_sumsq, in_parts, in_eps = scale.sumsq, scale.sumsq.shape[0], float(scale.eps)
    scaled = sumsq = None
    if resid is not None:
        sumsq = torch.empty((-(-N // 128) * sk, ld), dtype=torch.float32, device=x.device)
        if gamma is not None:
            if gamma.numel() != N or gamma.dtype not in (torch.float32, torch.bfloat16):
                return None
            scaled = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    st = _dev_state(x.device)
    f = _fn("gemm_bf16", "gf_gemm_bf16_tc_ex",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
             c_int, c_int, c_void_p, c_void_p, c_void_p,
             c_void_p, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    rc = f(_p(x), x.stride(0), _p(weight), _p(bias_f32), _p(out), cols, M, N, K, int(epi),
           1 if out_dtype == torch.float32 else 0, sk, _p(ws), _p(st["err"]), _stream(),
           _p(in_sumsq), in_parts, ld, in_eps, _p(resid), _p(scaled), _p(gamma),
           1 if gamma is not None and gamma.dtype == torch.float32 else 0, _p(sumsq))
    if rc in (-6, -7):
        return None
    _ok(rc, "gemm_bf16_tc")
    return out if resid is None else (out, scaled, sumsq)


# The residual epilogue takes the token tiles of decode steps.
RESID_MAX_TOKENS = 64

# The largest token count the gated product runs here for.  In a CUDA graph, 1.5B shapes, weights
# from HBM, two K splits (us, here / cuBLAS + SiLU*mul): 8 tokens 11.2 / 12.7, 16 tokens 11.9 / 12.9,
# 32 tokens 12.7 / 13.2, 48 tokens 13.2 / 13.3, 64 tokens 14.2 / 14.0 (one split: 20.5: a CTA's ring
# holds four 16 KB weight tiles beside the 8 KB token tiles, and two CTAs an SM keep twice as many
# bytes under way).  Inside a decode step of 4 layers the kernel up to 64 tokens, for the gated
# and the down product, takes 312 / 365 / 352 us at batch 32 / 48 / 64 against 323 / 370 / 362 with
# cuBLAS from 17 tokens on: it starts while the kernel before it runs and has its first weights
# by then, which a library kernel does not.
MAX_TOKENS = 64


def plain_limit(weight) -> int:
    """The largest token count for which a plain product with ``weight`` runs here."""
    return PLAIN_MAX_TOKENS_LONG_K if weight.shape[1] >= LONG_K else PLAIN_MAX_TOKENS


def try_linear(x, weight, bias_f32, out_dtype):
    """Run the tcgen05 kernel where it is the faster one (the small batches of decode steps and
    short prompt portions); ``None`` hands the product to cuBLAS."""
    if x.shape[0] > plain_limit(weight):
        return None
    return gemm(x, weight, bias_f32, out_dtype, epi=0)


# Plain products leave for cuBLAS above this many tokens.  In a CUDA graph on a B200, 1.5B shapes,
# weights from HBM (us, here / cuBLAS): q/k/v 8 tokens 4.2 / 5.6, 16 tokens 4.6 / 4.6, 32 tokens
# 6.3 / 4.6; output 4.3 / 5.0, 4.7 / 4.6, 6.5 / 4.5; down (a reduction of 8,960) 8 tokens 8.6 / 16.9,
# 32 tokens 10.6 / 13.4, 48 tokens 12.4 / 13.6, 64 tokens 13.8 / 13.7; q/k/v and output at 64 tokens
# 6.8 / 5.0 and 6.5 / 4.8 (their epilogue, the reduction of the K splits, grows with the tokens).
PLAIN_MAX_TOKENS = 16
PLAIN_MAX_TOKENS_LONG_K = 64   # for reductions of at least LONG_K
LONG_K = 4096
