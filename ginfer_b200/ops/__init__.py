"""Python face of the hand-written CUDA kernels.

Every function here launches a kernel from ``csrc/`` on the current CUDA stream (matrix products
of the bf16 path may go to cuBLAS, as the reference's do:
``ginfer/core/op/kernels/cuda/gemm_kernel/gemm_kernel.cu:93-156``).  There is no CPU path: a
tensor that is not on a CUDA device is an error, and so is a library that cannot be built.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_void_p

import torch

from .build import BuildError, build_all, load_library, set_pdl  # noqa: F401

_CODES = {torch.float32: 0, torch.bfloat16: 1}


def _code(dt: torch.dtype) -> int:
    try:
        return _CODES[dt]
    except KeyError:
        raise TypeError(f"kernels take float32 or bfloat16 activations, not {dt}") from None


def _p(t):
    """The device address of a tensor for a kernel (``None`` stays ``None``).  A tensor that is
    not on a CUDA device is refused here: its address would mean nothing to a kernel."""
    if t is None:
        return None
    if not t.is_cuda:
        raise RuntimeError("ginfer_b200 kernels run on a CUDA device only; got a tensor on "
                           f"{t.device}")
    return c_void_p(t.data_ptr())


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("ginfer_b200 kernels run on a CUDA device only; got a tensor on "
                               f"{t.device}")


def _ok(rc: int, what: str):
    if rc > 0:
        raise RuntimeError(f"{what}: CUDA error {rc} at launch")
    if rc < 0:
        raise RuntimeError(f"{what}: the kernel refused its arguments (code {rc})")


class _Counter:
    """Kernel launches made through this module (each entry point launches one kernel unless it
    says otherwise); read by the benchmark."""
    launches = 0


_fns: dict = {}


def _fn(lib_name: str, fn_name: str, argtypes, defines=(), kernels: int = 1):
    key = (lib_name, tuple(defines), fn_name)
    g = _fns.get(key)
    if g is None:
        lib = load_library(lib_name, tuple(defines))
        f = getattr(lib, fn_name)
        f.argtypes = argtypes
        f.restype = c_int

        def g(*args, _f=f, _k=kernels):
            _Counter.launches += _k
            return _f(*args)
        _fns[key] = g
    return g


def launch_count() -> int:
    return _Counter.launches


# ----------------------------------------------------------------------------- embedding
def embedding(token_ids: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    _cuda(token_ids, weight)
    assert token_ids.dtype == torch.int32 and token_ids.is_contiguous()
    T, (V, H) = token_ids.numel(), weight.shape
    out = torch.empty((T, H), dtype=weight.dtype, device=weight.device)
    f = _fn("elementwise", "gf_embedding",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _ok(f(_p(token_ids), _p(weight), _p(out), T, H, _code(weight.dtype), _stream()), "embedding")
    return out


# ----------------------------------------------------------------------------- add + rmsnorm
def add_rmsnorm(x: torch.Tensor, delta, gamma: torch.Tensor, eps: float, rows=None,
                want_sum: bool = True, out_dtype=None):
    """``s = x + delta`` in fp32; returns ``(s or None, s * gamma / rms(s))``.  ``x`` is the fp32
    residual stream or an activation; ``delta`` and the normed output have the activation dtype
    (``out_dtype``, else that of ``delta``, else of ``x``).  Without ``delta`` and ``rows`` the
    returned ``s`` is ``x`` itself."""
    _cuda(x, delta, gamma, rows)
    assert x.dim() == 2 and x.is_contiguous()
    H = x.shape[1]
    act = out_dtype or (x.dtype if delta is None else delta.dtype)
    if delta is not None:
        assert delta.shape == x.shape and delta.is_contiguous()
    assert gamma.numel() == H and gamma.is_contiguous()
    R = x.shape[0] if rows is None else rows.numel()
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.is_contiguous()
    normed = torch.empty((R, H), dtype=act, device=x.device)
    s = None
    if want_sum:
        if delta is None and rows is None:
            s = x
        elif delta is None:
            s = x.index_select(0, rows.long())
        else:
            s = torch.empty((R, H), dtype=torch.float32, device=x.device)
    f = _fn("elementwise", "gf_add_rmsnorm",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_int, c_void_p])
    sum_ptr = _p(s) if (want_sum and delta is not None) else None
    _ok(f(_p(x), _code(x.dtype), _p(delta), _p(gamma), _code(gamma.dtype), float(eps), _p(rows),
          sum_ptr, _p(normed), R, H, _code(act), _stream()), "add_rmsnorm")
    return s, normed


# ----------------------------------------------------------------------------- rope + KV write
def rope_kv_write(qkv: torch.Tensor, table, rotary_dim: int, positions: torch.Tensor,
                  slot_mapping, pages: torch.Tensor, nh: int, nkv: int, hd: int) -> None:
    """Rotate the q and k heads of ``qkv [T, (nh + 2 nkv) hd]`` (q in place) and, when
    ``slot_mapping`` is given, write k and v into ``pages [2, num_pages, page, nkv, hd]``."""
    _cuda(qkv, table, positions, slot_mapping, pages)
    assert qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] == (nh + 2 * nkv) * hd
    assert pages.is_contiguous() and pages.dtype == qkv.dtype and pages.shape[0] == 2
    assert tuple(pages.shape[3:]) == (nkv, hd)
    if table is not None:
        assert table.dtype == torch.float32 and table.is_contiguous()
        assert table.shape[1] == rotary_dim and rotary_dim % 2 == 0 and rotary_dim <= hd
    T = qkv.shape[0]
    f = _fn("elementwise", "gf_rope_kv_write",
            [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
             c_int, c_int, c_int, c_int, c_void_p])
    _ok(f(_p(qkv), qkv.stride(0), _p(table), int(rotary_dim), _p(positions), _p(slot_mapping),
          _p(pages[0]), _p(pages[1]), T, nh, nkv, hd, _code(qkv.dtype), _stream()),
        "rope_kv_write")


# ----------------------------------------------------------------------------- silu * up
def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """``gate_up [T, 2 I]`` with gate and up interleaved (g0, u0, g1, u1, ...) -> ``[T, I]``."""
    _cuda(gate_up)
    assert gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.shape[1] % 2 == 0
    T, I = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty((T, I), dtype=gate_up.dtype, device=gate_up.device)
    f = _fn("elementwise", "gf_silu_mul", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _ok(f(_p(gate_up), _p(out), T, I, _code(gate_up.dtype), _stream()), "silu_mul")
    return out


# ----------------------------------------------------------------------------- attention
def paged_attention_simt(qkv, pages, block_table, seq_of_token, positions, nh, nkv, hd, scale,
                         window, page_size):
    _cuda(qkv, pages, block_table, seq_of_token, positions)
    T = qkv.shape[0]
    out = torch.empty((T, nh * hd), dtype=qkv.dtype, device=qkv.device)
    f = _fn("attention_simt", "gf_paged_attention_simt",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p])
    rc = f(_p(qkv), qkv.stride(0), _p(pages[0]), _p(pages[1]), _p(block_table),
           block_table.stride(0), _p(seq_of_token), _p(positions), _p(out), T, nh, nkv, hd,
           page_size, int(window), float(scale), _code(qkv.dtype), _stream())
    if rc == -3:
        raise ValueError(f"attention kernels take head sizes up to 256 and head counts that are "
                         f"a multiple of the kv head count; got head_dim={hd}, heads={nh}, "
                         f"kv_heads={nkv}")
    _ok(rc, "paged_attention_simt")
    return out


def attention_fuses_rope(qkv: torch.Tensor, ctx, nh: int, nkv: int, hd: int) -> bool:
    """True if :func:`paged_attention` can rotate q and k and write the new k and v itself for
    this step (pass ``rope=`` then, and skip :func:`rope_kv_write`)."""
    from . import attention_bf16
    return attention_bf16.fuses_rope(qkv, ctx, hd, nh, nkv)


def paged_attention(qkv: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor, ctx,
                    nh: int, nkv: int, hd: int, scale: float, window: int, page_size: int,
                    rope=None) -> torch.Tensor:
    """Attention of the step's queries (first ``nh * hd`` columns of ``qkv``) over the paged
    cache; returns ``[T, nh * hd]``.  Picks the kernel by dtype, head size and batch shape.
    ``rope = (table or None, rotary_dim, write)`` where :func:`attention_fuses_rope`: q and k are
    still unrotated and the new k and v not yet in the cache."""
    from . import attention_bf16
    if qkv.dtype == torch.bfloat16:
        out = attention_bf16.try_run(qkv, pages, block_table, ctx, nh, nkv, hd, scale, window,
                                     page_size, rope=rope)
        if out is not None:
            return out
    assert rope is None
    return paged_attention_simt(qkv, pages, block_table, ctx.seq_of_token, ctx.positions, nh, nkv,
                                hd, scale, window, page_size)


# ----------------------------------------------------------------------------- sampling
_argmax_scratch: dict = {}


def argmax(logits: torch.Tensor) -> torch.Tensor:
    _cuda(logits)
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous()
    R, V = logits.shape
    out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    words = 2 * R * (-(-V // 4096))
    if torch.cuda.is_current_stream_capturing():
        scratch = torch.empty(words, dtype=torch.int32, device=logits.device)
    else:
        scratch = _argmax_scratch.get(logits.device)
        if scratch is None or scratch.numel() < words:
            scratch = torch.empty(max(words, 1 << 16), dtype=torch.int32, device=logits.device)
            _argmax_scratch[logits.device] = scratch
    f = _fn("sampling", "gf_argmax", [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p])
    rc = f(_p(logits), _p(out), R, V, _p(scratch), _stream())
    if rc == -5:
        raise ValueError(f"argmax takes at most 4096 rows at a time, got {R}")
    _ok(rc, "argmax")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """Row ``r``: arg-max if ``temperature[r] <= 0`` else the first index whose cumulative
    ``softmax(logits / temperature)`` reaches ``u[r]``."""
    _cuda(logits, temperature, u)
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous()
    R, V = logits.shape
    assert temperature.dtype == torch.float32 and u.dtype == torch.float32
    assert temperature.numel() == R and u.numel() == R
    out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    f = _fn("sampling", "gf_sample",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _ok(f(_p(logits), _p(temperature), _p(u), _p(out), R, V, _stream()), "sample")
    return out


def scatter_tokens(dst: torch.Tensor, dst_idx: torch.Tensor, src: torch.Tensor,
                   src_idx: torch.Tensor) -> None:
    """``dst[dst_idx[i]] = src[src_idx[i]]`` (all int32, on the device)."""
    _cuda(dst, dst_idx, src, src_idx)
    assert all(t.dtype == torch.int32 for t in (dst, dst_idx, src, src_idx))
    n = dst_idx.numel()
    assert src_idx.numel() == n
    f = _fn("sampling", "gf_scatter_tokens",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _ok(f(_p(dst), _p(dst_idx), _p(src), _p(src_idx), n, _stream()), "scatter_tokens")


def qkv_rope_write(x, linear, table, rot, positions, slot_mapping, pages, nh, nkv, hd):
    """``linear(x)`` with q and k rotated and k and v written to the cache by the product's own
    epilogue, where that is served (bf16, many tokens; see ``gemm_prefill.qkv_rope_write``), else
    ``None``."""
    if (getattr(linear, "dtype", None) != torch.bfloat16 or x.dtype != torch.bfloat16
            or linear.out_dtype != torch.bfloat16):
        return None
    from . import gemm_prefill
    return gemm_prefill.qkv_rope_write(x, linear.weight, linear._bias_f32, table, rot, positions,
                                       slot_mapping, pages, nh, nkv, hd)


from .linear import GatedLinear, Linear, add_to  # noqa: E402,F401
