"""Matrix products ``y = x W^T (+ b)`` with ``W [out, in]`` as Hugging Face stores it (the
reference reads the same memory as a column-major ``[in, out]`` view:
``ginfer/core/layer/linear.cc:13-16``).

float32: the hand-written FMA kernel of ``csrc/gemm_f32.cu`` (no reduced-precision mode).
bfloat16: the tcgen05 kernels of ``csrc/gemm_bf16.cu`` (few tokens) and ``csrc/gemm_prefill.cu``
(the gated product of many tokens) where they are the faster ones, else cuBLAS through ``torch``
(fp32 accumulation), which is what the reference uses for every product.
"""
from __future__ import annotations

from ctypes import c_int, c_void_p

import torch

from . import _cuda, _fn, _ok, _p, _stream, silu_mul


def gemm_f32(x: torch.Tensor, w: torch.Tensor, bias=None) -> torch.Tensor:
    _cuda(x, w, bias)
    assert x.dtype == torch.float32 and w.dtype == torch.float32
    assert x.dim() == 2 and w.dim() == 2 and x.stride(1) == 1 and w.is_contiguous()
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == N
    out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    f = _fn("gemm_f32", "gf_gemm_f32",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _ok(f(_p(x), x.stride(0), _p(w), _p(bias), _p(out), N, M, N, K, _stream()), "gemm_f32")
    return out


class Linear:
    """``y = x W^T + b``.  ``out_dtype`` float32 asks for fp32 results from bf16 operands (the
    output head)."""

    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None = None,
                 out_dtype: torch.dtype | None = None):
        _cuda(weight, bias)
        self.weight = weight.contiguous()
        self.bias = bias
        self.out_features, self.in_features = weight.shape
        self.dtype = weight.dtype
        self.out_dtype = out_dtype or weight.dtype
        if self.dtype == torch.float32:
            if bias is not None:
                self.bias = bias.float().contiguous()
        elif self.dtype == torch.bfloat16:
            # cuBLAS adds the bias in its fp32 epilogue; it wants the operands' dtype
            self._bias_lib = None if bias is None else bias.to(torch.bfloat16).contiguous()
            self._bias_f32 = None if bias is None else bias.float().contiguous()
        else:
            raise TypeError(f"Linear takes float32 or bfloat16 weights, not {self.dtype}")

    def __call__(self, x) -> torch.Tensor:
        if hasattr(x, "materialize"):                 # a normalisation not computed yet
            if self.dtype == torch.bfloat16 and x.scaled is not None:
                from . import gemm_bf16
                y = gemm_bf16.gemm(x.scaled, self.weight, self._bias_f32, self.out_dtype,
                                   scale=gemm_bf16.RowScale(x.summed.sumsq, x.eps))
                if y is not None:
                    return y
            x = x.materialize()
        if x.dtype != self.dtype:
            raise TypeError(f"Linear holds {self.dtype} weights but got {x.dtype} input")
        if self.dtype == torch.float32:
            return gemm_f32(x, self.weight, self.bias)
        from . import gemm_bf16
        y = gemm_bf16.try_linear(x, self.weight, self._bias_f32, self.out_dtype)
        if y is not None:
            return y
        if self.out_dtype == torch.float32:
            y = torch.mm(x, self.weight.t(), out_dtype=torch.float32)
            if self._bias_f32 is not None:
                y += self._bias_f32
            return y
        if self._bias_lib is not None:
            return torch.addmm(self._bias_lib, x, self.weight.t())
        return torch.mm(x, self.weight.t())


def add_to(linear: "Linear", x: torch.Tensor, residual: torch.Tensor, gamma=None):
    """``(s, partial sums of squares of s's rows, s * gamma in bf16, gamma)`` with ``s = residual
    + linear(x)`` in fp32, from one kernel (the fields of ``parts.base.Summed``), or ``None`` if
    the kernel does not serve this case (then the caller adds in the next norm).  ``gamma``: the
    weight of the RMS norm that follows, if it can be folded."""
    if linear.dtype != torch.bfloat16 or residual.dtype != torch.float32:
        return None
    from . import gemm_bf16
    if x.shape[0] > gemm_bf16.plain_limit(linear.weight):
        return None
    got = gemm_bf16.gemm(x, linear.weight, linear._bias_f32, resid=residual, gamma=gamma)
    if got is None:
        return None
    s, scaled, sumsq = got
    return s, sumsq, scaled, gamma


# From this many tokens on the gated product runs on the persistent tcgen05 kernel of
# csrc/gemm_prefill.cu (on CTA pairs, SiLU*mul in its epilogue).  On a B200 in a CUDA graph, against
# cuBLAS + the SiLU*mul kernel: at the 1.5B shape (17920 x 1536) 512 tokens 26.9 against 26.6 us,
# 768 tokens 36.2 against 37.9, 1,024 tokens 45.8 against 48.8, 2,048 tokens 84.6 against 96.0,
# 8,192 tokens 304 against 386; at the 7B shape (37888 x 3584) 768 tokens 151 against 153, 1,024
# tokens 193 against 210, 2,048 tokens 367 against 392.
PREFILL_GATED_MIN_TOKENS = 768


def _gemm_bf16():
    from . import gemm_bf16
    return gemm_bf16


class GatedLinear:
    """``silu(x W_g^T) * (x W_u^T)``.  The two matrices are joined row by row (gate_0, up_0,
    gate_1, up_1, ...) so that ``x`` is read once and a gate meets its up value in neighbouring
    accumulator rows: the tcgen05 kernel combines them in its epilogue and writes only the
    product.  Gate and up are rounded to the activation dtype before they are combined, whichever
    kernel runs, so the result does not depend on the kernel chosen."""

    def __init__(self, gate: torch.Tensor, up: torch.Tensor):
        assert gate.shape == up.shape and gate.dtype == up.dtype
        self.intermediate, k = gate.shape
        self.proj = Linear(torch.stack([gate, up], dim=1).reshape(2 * self.intermediate, k))

    def __call__(self, x) -> torch.Tensor:
        if hasattr(x, "materialize"):                 # a normalisation not computed yet
            if self.proj.dtype == torch.bfloat16 and x.scaled is not None \
                    and x.scaled.shape[0] <= _gemm_bf16().MAX_TOKENS:
                gb = _gemm_bf16()
                z = gb.gemm(x.scaled, self.proj.weight, None, torch.bfloat16, epi=2,
                            scale=gb.RowScale(x.summed.sumsq, x.eps))
                if z is not None:
                    return z
            x = x.materialize()
        if x.dtype == torch.bfloat16:
            from . import gemm_bf16, gemm_prefill
            if x.shape[0] <= gemm_bf16.MAX_TOKENS:
                z = gemm_bf16.gemm(x, self.proj.weight, None, torch.bfloat16, epi=2)
                if z is not None:
                    return z
            elif x.shape[0] >= PREFILL_GATED_MIN_TOKENS:
                z = gemm_prefill.gemm(x, self.proj.weight, None, torch.bfloat16, epi=2)
                if z is not None:
                    return z
        return silu_mul(self.proj(x))
