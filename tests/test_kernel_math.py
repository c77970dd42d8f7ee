"""Arithmetic that kernels do in an unusual way, restated on the host with the constants read from
the CUDA sources, so that the bounds their comments give are checked where no GPU is needed."""
import os
import re

import numpy as np

CSRC = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "ginfer_b200", "csrc")


def test_cubic_exp2_of_the_prefill_attention_keeps_its_bound():
    """``poly_exp2`` (``attention_tc.cu``): 2^x as 2^n * p(f), n the nearest integer taken from
    the mantissa of x + 1.5 * 2^23, f = x - n in [-0.5, 0.5], p a cubic; in float32 as the
    kernel computes it.  Its comment promises 7.5e-5 relative; inputs are clamped at -125, above
    which every result is a normal number."""
    src = open(os.path.join(CSRC, "attention_tc.cu")).read()
    body = src[src.index("float poly_exp2(float x)"):]
    body = body[:body.index("}")]
    c3, c2, c1, c0 = (np.float32(v) for v in re.findall(r"(\d\.\d+)f", body)[-4:])
    magic = np.float32(12582912.0)
    assert "12582912.f" in body and "-125.f" in body
    x = np.concatenate([np.linspace(-125, 8, 400001), np.arange(-125, 9), [-1e4, -200.0]])
    x = np.maximum(x.astype(np.float32), np.float32(-125))
    t = x + magic
    f = x - (t - magic)
    assert np.abs(f).max() <= 0.5
    p = ((c3 * f + c2) * f + c1) * f + c0
    assert p.dtype == np.float32
    got = (p.view(np.int32) + (t.view(np.int32) << np.int32(23))).view(np.float32)
    want = np.exp2(x.astype(np.float64))
    assert np.abs(got / want - 1).max() < 7.6e-5
    assert np.all(np.diff(got[:400001]) >= 0)          # monotonic over the whole range
