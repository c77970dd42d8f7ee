"""bf16 matrix products on the 5th-generation tensor cores (``csrc/gemm_bf16.cu``)."""
from __future__ import annotations


def try_linear(x, weight, bias_f32, out_dtype):
    """Run the tcgen05 kernel if it takes this shape; ``None`` hands the product to cuBLAS."""
    return None
