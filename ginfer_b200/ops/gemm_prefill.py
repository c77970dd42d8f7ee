"""bf16 matrix products for many tokens (``csrc/gemm_prefill.cu``): a persistent tcgen05 kernel
with two accumulators in tensor memory, so that a tile's epilogue (bias, or SiLU*mul over
interleaved gate/up rows, or bias + rotation + cache write for the joined q/k/v product) runs
while the next tile is multiplied."""
from __future__ import annotations

import os
from ctypes import c_int, c_void_p

import torch


def supports(x: torch.Tensor, weight: torch.Tensor) -> bool:
    K = weight.shape[1]
    return (K % 8 == 0 and x.dim() == 2 and x.stride(1) == 1 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0 and weight.is_contiguous())


# GINFER_B200_GEMM_PAIR=0: the products of many tokens on single CTAs instead of CTA pairs
PAIR = os.environ.get("GINFER_B200_GEMM_PAIR", "1") != "0"


def gemm(x, weight, bias_f32=None, out_dtype=torch.bfloat16, epi: int = 0, ctas: int = 0,
         pair: bool | None = None):
    """``x [M, K] @ weight[N, K]^T``; ``epi`` 0: (+ bias) -> ``[M, N]``; ``epi`` 2: weight rows
    are interleaved (gate_i, up_i) and the result is ``silu(gate) * up`` -> ``[M, N / 2]``.
    ``ctas``: CTAs to launch (0: one an SM).  ``pair``: on CTA pairs (tiles of 256 tokens x 256
    weight rows, tcgen05 ``cta_group::2``; ``None``: the default).  ``None`` if the kernel cannot
    serve the shape."""
    from . import _cuda, _fn, _ok, _p, _stream
    from .gemm_bf16 import error_word
    if not supports(x, weight):
        return None
    _cuda(x, weight, bias_f32)
    M, K = x.shape
    N = weight.shape[0]
    cols = N // 2 if epi == 2 else N
    out = torch.empty((M, cols), dtype=out_dtype, device=x.device)
    if M == 0:
        return out
    f = _fn("gemm_prefill", "gf_gemm_prefill",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
             c_int, c_int, c_void_p, c_void_p, c_int])
    rc = f(_p(x), x.stride(0), _p(weight), _p(bias_f32), _p(out), cols, M, N, K, int(epi),
           1 if out_dtype == torch.float32 else 0, int(ctas), _p(error_word(x.device)), _stream(),
           1 if (PAIR if pair is None else pair) else 0)
    if rc == -6:
        return None
    _ok(rc, "gemm_prefill")
    return out


# The joined q/k/v product with the rotation and the cache write in its epilogue is an option
# (GINFER_B200_QKV_EPILOGUE=1, then from QKV_MIN_TOKENS tokens on), not the default: cuBLAS with the
# rotation kernel behind it is the faster pair.  On a B200, in a prompt step of 4 layers and the head
# from a CUDA graph (us, epilogue / cuBLAS + rotation kernel): 1.5B shape 1,024 tokens 793 / 759,
# 1,536 tokens 909 / 887, 2,048 tokens 1,092 / 1,083, 4,096 tokens 1,914 / 1,895; 7B shape 1,024 tokens
# 1,960 / 1,942, 2,048 tokens 3,373 / 3,381, 4,096 tokens 6,623 / 6,575; the whole step of 2,048 tokens
# at the 1.5B shape 5.70 / 5.65 ms, a 32,768-token prompt in portions 216 / 214 ms, the reference's
# throughput run level; only the serving run of 64 requests, whose steps mix portions of prompts
# with decoded tokens, is faster with it (0.676 / 0.686 s).  Alone at 2,048 tokens the kernel takes 19.3 us against 11.7 + 4.6:
# its 128 tiles are one round for 148 CTAs, so its epilogue hides behind nothing, and where it has
# several rounds its products are behind cuBLAS's (44 against 37.5 us at 8,192 tokens).
QKV_MIN_TOKENS = 1024
QKV_EPILOGUE = os.environ.get("GINFER_B200_QKV_EPILOGUE", "0") != "0"


def qkv_epilogue_serves(x, weight, table, rot, positions, slot_mapping, pages, nh, nkv, hd,
                        min_tokens: int) -> bool:
    """Whether :func:`qkv_rope_write` takes this case: at least ``min_tokens`` tokens, head sizes 64
    and 128 with the whole head rotated, a run that writes its cache, bf16 operands and pages,
    an fp32 table, int32 positions and slots."""
    M = x.shape[0]
    return not (M < min_tokens or hd not in (64, 128) or table is None or rot != hd
                or slot_mapping is None or x.dtype != torch.bfloat16 or not supports(x, weight)
                or weight.dtype != torch.bfloat16
                or weight.shape[0] != (nh + 2 * nkv) * hd or table.dtype != torch.float32
                or not table.is_contiguous() or table.shape[1] != hd or table.data_ptr() % 16
                or pages.dtype != torch.bfloat16 or not pages.is_contiguous()
                or pages.shape[0] != 2 or tuple(pages.shape[3:]) != (nkv, hd)
                or positions.dtype != torch.int32 or slot_mapping.dtype != torch.int32
                or not positions.is_contiguous() or not slot_mapping.is_contiguous()
                or positions.numel() < M or slot_mapping.numel() < M)


def qkv_rope_write(x, weight, bias_f32, table, rot, positions, slot_mapping, pages, nh, nkv, hd,
                   min_tokens: int | None = None, ctas: int = 0):
    """The q/k/v product of a step of many tokens with bias, the rotation of q and k and the write
    of k and v to the paged cache in its epilogue (what :func:`ginfer_b200.ops.rope_kv_write`
    does behind a plain product).  ``pages [2, num_pages, page, nkv, hd]`` bf16.  Returns
    ``[T, (nh + 2 nkv) hd]`` with q and k rotated, or ``None`` if the kernel does not serve the
    case (:func:`qkv_epilogue_serves`; ``min_tokens`` is ``QKV_MIN_TOKENS`` unless given)."""
    from . import _cuda, _fn, _ok, _p, _stream
    from .gemm_bf16 import error_word
    M, K = x.shape
    if min_tokens is None:
        if not QKV_EPILOGUE:
            return None
        min_tokens = QKV_MIN_TOKENS
    if not qkv_epilogue_serves(x, weight, table, rot, positions, slot_mapping, pages, nh, nkv, hd,
                               min_tokens):
        return None
    _cuda(x, weight, bias_f32, table, positions, slot_mapping, pages)
    out = torch.empty((M, weight.shape[0]), dtype=torch.bfloat16, device=x.device)
    f = _fn("gemm_prefill", "gf_gemm_prefill_qkv",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
             c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p])
    rc = f(_p(x), x.stride(0), _p(weight), _p(bias_f32), _p(out), out.stride(0), M, K, nh, nkv,
           hd, _p(table), _p(positions), _p(slot_mapping), _p(pages[0]), _p(pages[1]), int(ctas),
           _p(error_word(x.device)), _stream())
    if rc == -6:
        return None
    _ok(rc, "gemm_prefill_qkv")
    return out
