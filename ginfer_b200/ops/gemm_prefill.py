"""bf16 matrix products for many tokens (``csrc/gemm_prefill.cu``): a persistent tcgen05 kernel
with two accumulators in tensor memory, so that a tile's epilogue (bias, or SiLU*mul over
interleaved gate/up rows) runs while the next tile is multiplied."""
from __future__ import annotations

from ctypes import c_int, c_void_p

import torch


def supports(x: torch.Tensor, weight: torch.Tensor) -> bool:
    K = weight.shape[1]
    return (K % 8 == 0 and x.dim() == 2 and x.stride(1) == 1 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0 and weight.is_contiguous())


def gemm(x, weight, bias_f32=None, out_dtype=torch.bfloat16, epi: int = 0, ctas: int = 0):
    """``x [M, K] @ weight[N, K]^T``; ``epi`` 0: (+ bias) -> ``[M, N]``; ``epi`` 2: weight rows
    are interleaved (gate_i, up_i) and the result is ``silu(gate) * up`` -> ``[M, N / 2]``.
    ``ctas``: CTAs to launch (0: one an SM).  ``None`` if the kernel cannot serve the shape."""
    from . import _fn, _ok, _p, _stream
    from .gemm_bf16 import error_word
    if not supports(x, weight):
        return None
    M, K = x.shape
    N = weight.shape[0]
    cols = N // 2 if epi == 2 else N
    out = torch.empty((M, cols), dtype=out_dtype, device=x.device)
    if M == 0:
        return out
    f = _fn("gemm_prefill", "gf_gemm_prefill",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
             c_int, c_int, c_void_p, c_void_p])
    rc = f(_p(x), x.stride(0), _p(weight), _p(bias_f32), _p(out), cols, M, N, K, int(epi),
           1 if out_dtype == torch.float32 else 0, int(ctas), _p(error_word(x.device)), _stream())
    if rc == -6:
        return None
    _ok(rc, "gemm_prefill")
    return out
