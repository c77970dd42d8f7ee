"""The decode-attention entry point that allocates nothing (``gf_attn_decode_static``), called
through its exported C symbol as a program without PyTorch would call it.

Some users of the library cannot call cudaMalloc at the point where they need attention: their
process gave all device memory to its own pools at start-up, or it runs a loop that must not take
the allocator's locks.  For them the library carries the scratch of the split-KV decode kernel in
its own device image.  This file checks that the entry point gives what the regular one gives (the
one whose scratch the caller passes), twice in a row on different inputs (the array is shared and
keeps the last call's contents), and that a call too large for the array is refused with a text
that says so.  It is collected last, and it passes alone in a fresh process as well as after the
other tests.
"""
import ctypes
import gc
import math
from ctypes import c_char_p, c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HD = 64


def _library():
    from ginfer_b200.ops.build import compile_library
    lib = ctypes.CDLL(compile_library("attention_bf16", (f"GF_HEAD_DIM={HD}",)))
    f = lib.gf_attn_decode_static
    f.restype = c_int
    f.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                  c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p]
    lib.gf_attn_decode_static_error.restype = c_char_p
    lib.gf_attn_decode_static_error.argtypes = []
    return lib


def _case(seed, lens, nh, nkv, page):
    g = torch.Generator(device="cpu").manual_seed(seed)
    B = len(lens)
    need = sum(-(-n // page) for n in lens)
    perm = torch.randperm(need + 3, generator=g)
    width = max(-(-n // page) for n in lens)
    table = torch.full((B, width), -1, dtype=torch.int32)
    at = 0
    for b, n in enumerate(lens):
        k = -(-n // page)
        table[b, :k] = perm[at:at + k].to(torch.int32)
        at += k
    pages = torch.randn(2, need + 3, page, nkv, HD, generator=g).to(torch.bfloat16)
    qkv = torch.randn(B, (nh + 2 * nkv) * HD, generator=g).to(torch.bfloat16)
    return dict(qkv=qkv.to(DEV), pages=pages.to(DEV), table=table.to(DEV),
                cu=torch.arange(B + 1, dtype=torch.int32, device=DEV),
                positions=torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV))


def _static(lib, c, nh, nkv, page, window, splits, check_device=True):
    B = c["qkv"].shape[0]
    out = torch.full((B, nh * HD), float("nan"), dtype=torch.bfloat16, device=DEV)
    gc.collect()            # tensors that earlier tests left in cycles go now, not during the call
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated(DEV), torch.cuda.memory_reserved(DEV)
    free_before = torch.cuda.mem_get_info(DEV)[0]          # the driver's own count of free bytes
    rc = lib.gf_attn_decode_static(
        c["qkv"].data_ptr(), c["qkv"].stride(0), c["pages"][0].data_ptr(),
        c["pages"][1].data_ptr(), c["table"].data_ptr(), c["table"].stride(0),
        c["cu"].data_ptr(), c["positions"].data_ptr(), out.data_ptr(), B, nh, nkv, page, window,
        1.0 / math.sqrt(HD), splits, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    # the call took nothing from PyTorch's allocator, and nothing from the device behind its back
    # (a cudaMalloc inside the library would show in the driver's count; the first call of a
    # process may load the kernel's module, so the caller makes one call before it counts)
    assert (torch.cuda.memory_allocated(DEV), torch.cuda.memory_reserved(DEV)) == before
    if check_device:
        assert torch.cuda.mem_get_info(DEV)[0] == free_before
    return rc, out


def test_static_scratch_entry_point_matches_the_regular_one_twice_in_a_row():
    from ginfer_b200.ops import attention_bf16
    lib = _library()
    nh, nkv, page = 6, 2, 16
    warm = _case(0, [30, 50], nh, nkv, page)
    _static(lib, warm, nh, nkv, page, 0, 3, check_device=False)      # loads what a first call loads
    for seed, lens, window, splits in [(1, [700, 90, 1, 333], 0, 7), (2, [64, 1500, 257], 100, 5),
                                       (3, [40, 41], 0, 1), (4, [900, 12, 77], 0, 8)]:
        c = _case(seed, lens, nh, nkv, page)
        rc, got = _static(lib, c, nh, nkv, page, window, splits)
        assert rc == 0, lib.gf_attn_decode_static_error()
        # the regular entry point with a scratch buffer of the caller's runs the same kernel with
        # the same splits: the same bits
        same = attention_bf16.decode(c["qkv"], c["pages"], c["table"], c["cu"], c["positions"],
                                     len(lens), nh, nkv, HD, 1.0 / math.sqrt(HD), window, page,
                                     splits, through_scratch=True, use_tma=False)
        assert torch.equal(got, same)
        # and the path serving takes (tiles by TMA, splits merged inside a cluster) agrees
        want = attention_bf16.decode(c["qkv"], c["pages"], c["table"], c["cu"], c["positions"],
                                     len(lens), nh, nkv, HD, 1.0 / math.sqrt(HD), window, page,
                                     splits)
        torch.testing.assert_close(got.float(), want.float(), atol=1e-2, rtol=2e-2)
        assert not torch.isnan(got.float()).any()


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    lib = _library()
    nh, nkv, page = 32, 2, 16
    c = _case(4, [100] * 64, nh, nkv, page)
    _static(lib, _case(0, [30, 50], nh, nkv, page), nh, nkv, page, 0, 3, check_device=False)
    rc, out = _static(lib, c, nh, nkv, page, 0, 16)     # 64 * 32 * 16 * 66 * 4 bytes = 8.6 MB
    torch.cuda.synchronize()
    assert rc == -8
    msg = lib.gf_attn_decode_static_error().decode()
    assert "8650752" in msg and "4194304" in msg and "64 requests" in msg
    assert torch.isnan(out.float()).all()                # nothing was launched
    rc, out = _static(lib, c, nh, nkv, page, 0, 4)       # a quarter of the splits fits
    torch.cuda.synchronize()
    assert rc == 0 and lib.gf_attn_decode_static_error() == b""
    assert not torch.isnan(out.float()).any()
