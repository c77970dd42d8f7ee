"""bf16 attention kernels for the serving path (``csrc/attention_bf16.cu``): split-KV decode and
tensor-core prefill over the paged cache.  The library is compiled for the model's head size."""
from __future__ import annotations

import os
from ctypes import c_float, c_int, c_void_p

import torch

KEY_TILE = 64
CTAS_PER_SM = 2                # resident CTAs of the decode kernel on one SM
MAX_SPLITS = 64

_scratch: dict = {}


def supports(hd: int, nh: int, nkv: int) -> bool:
    return hd % 16 == 0 and 16 <= hd <= 256 and nh % nkv == 0


def decode_splits(batch: int, nh: int, nkv: int, max_keys: int, sms: int | None = None) -> int:
    """How many ways to split each request's keys so that the grid fills the GPU without a second
    wave: a power of two up to 8, so that the splits of a request can form a thread-block cluster.  ``sms``: the
    device's SM count (asked of the current device if ``None``)."""
    from .gemm_bf16 import num_sms
    chunks = (nh // nkv + 15) // 16
    base = max(1, batch * nkv * chunks)
    target = (sms or num_sms()) * CTAS_PER_SM
    want = min(max(1, target // base), max(1, -(-max_keys // KEY_TILE)))
    splits = 1
    while splits * 2 <= min(want, 8):                 # clusters of 16 schedule badly: 8 at most
        splits *= 2
    # (never more CTAs than fit at once: 48 requests in 4 splits, 384 CTAs for 296 places, measured
    # 17.3 us against 10.6 in 2)
    return splits


MAX_PARTS = 16                 # clusters that may share one request's keys
# the fewest keys a CTA should be left with: where one cluster a request leaves more than half of
# the SMs idle, and otherwise (the kernel that adds the parts up costs 3 us: 8 requests of 4,096
# keys measured 16.5 us in two parts against 12.0 in one, of 32,768 keys 46.9 against 58.2)
MIN_KEYS_PER_CTA_IDLE, MIN_KEYS_PER_CTA = 256, 1024


def decode_partition(batch: int, nh: int, nkv: int, max_keys: int,
                     sms: int | None = None) -> tuple[int, int]:
    """(splits, parts): how many CTAs form the cluster that merges through distributed shared
    memory, and how many such clusters share a request's keys (their results are added up by a
    second kernel).  More than one cluster only where 8 CTAs a request and kv head leave most of
    the GPU idle: few requests with many keys."""
    from .gemm_bf16 import num_sms
    splits = decode_splits(batch, nh, nkv, max_keys, sms)
    if splits < 8:
        return splits, 1
    chunks = (nh // nkv + 15) // 16
    base = max(1, batch * nkv * chunks)
    n_sms = sms or num_sms()
    least = MIN_KEYS_PER_CTA_IDLE if 2 * base * splits <= n_sms else MIN_KEYS_PER_CTA
    want = min(n_sms * CTAS_PER_SM // (base * splits), max_keys // (least * splits), MAX_PARTS)
    return splits, max(1, want)


def tma_serves(hd: int, page_size: int, splits: int) -> bool:
    """Whether decode attention takes the kernel that loads its tiles by TMA."""
    return (hd % 64 == 0 and page_size % 8 == 0 and splits in (1, 2, 4, 8, 16)
            and (KEY_TILE % page_size == 0 or page_size % KEY_TILE == 0))


def _scratch_for(nbytes: int, device) -> torch.Tensor:
    key = (device.index if device.index is not None else torch.cuda.current_device())
    buf = _scratch.get(key)
    if buf is None or buf.numel() * 4 < nbytes:
        buf = torch.empty(max(nbytes // 4 + 1, 1 << 20), dtype=torch.float32, device=device)
        _scratch[key] = buf
    return buf


def decode(qkv, pages, block_table, cu_seqlens_q, positions, B, nh, nkv, hd, scale, window,
           page_size, splits, out=None, scratch=None, through_scratch=False, rope=None,
           use_tma=True, stages=3, parts=1):
    """Split-KV decode attention.  ``splits`` of 2, 4, 8 or 16 merge inside a thread-block cluster
    (no scratch memory) unless ``through_scratch``; any other number goes through scratch.
    ``rope = (table or None, rotary_dim, write)``: q and k arrive unrotated and the kernel
    rotates them itself and (``write``) puts the new k and v into their cache slot.
    ``use_tma``: take the kernel that loads its tiles by TMA where it serves the case (head sizes
    64, 128, 192 and 256, page sizes 8, 16, 32, 64 and multiples of 64, cluster merge), with a
    ring of ``stages`` tiles (2 .. 6; three let two CTAs share an SM, and with clusters of 8 only
    that fits a grid of 128 CTAs in one wave: four and six stages measured half as fast).
    ``parts`` > 1 (TMA kernel only): that many clusters share a request's keys and a second kernel
    adds their results up (see :func:`decode_partition`)."""
    from . import _fn, _ok, _p, _stream
    defines = (f"GF_HEAD_DIM={hd}",)
    if out is None:
        out = torch.empty((qkv.shape[0], nh * hd), dtype=torch.bfloat16, device=qkv.device)
    if splits > 1 and scratch is None and (through_scratch or splits not in (2, 4, 8, 16)):
        nbytes = B * nh * splits * (hd + 2) * 4
        if torch.cuda.is_current_stream_capturing():
            # a graph keeps its own scratch (from the graph's memory pool): the shared buffer
            # may be replaced by a larger one later
            scratch = torch.empty(nbytes // 4, dtype=torch.float32, device=qkv.device)
        else:
            scratch = _scratch_for(nbytes, qkv.device)
    if use_tma and hd % 64 == 0 and scratch is None and not through_scratch:
        from .gemm_bf16 import error_word
        table, rot, write = rope if rope is not None else (None, 0, False)
        parts = max(1, int(parts))
        part_scratch = None
        if parts > 1:
            nbytes = B * nh * parts * (hd + 2) * 4
            if torch.cuda.is_current_stream_capturing():
                part_scratch = torch.empty(nbytes // 4, dtype=torch.float32, device=qkv.device)
            else:
                part_scratch = _scratch_for(nbytes, qkv.device)
        f = _fn("attention_bf16", "gf_attn_decode_tma",
                [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                 c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p,
                 c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p], defines, kernels=1)
        rc = f(_p(qkv), qkv.stride(0), _p(pages[0]), _p(pages[1]), pages.shape[1],
               _p(block_table), block_table.stride(0), _p(cu_seqlens_q), _p(positions), _p(out), B,
               nh, nkv, page_size, int(window), float(scale), int(splits),
               int(stages), _p(table),
               int(rot) if table is not None else 0, 1 if rope is not None else 0,
               int(bool(write)), _p(error_word(qkv.device)), _stream(), parts, _p(part_scratch))
        if rc == 0 and parts > 1:
            from . import _Counter
            _Counter.launches += 1                     # the kernel that adds the parts up
        if rc != -6:
            _ok(rc, "attn_decode_tma")
            return out
    if rope is not None:
        table, rot, write = rope
        f = _fn("attention_bf16", "gf_attn_decode_rope",
                [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                 c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p,
                 c_int, c_int, c_void_p], defines, kernels=1)
        _ok(f(_p(qkv), qkv.stride(0), _p(pages[0]), _p(pages[1]), _p(block_table),
              block_table.stride(0), _p(cu_seqlens_q), _p(positions), _p(out), _p(scratch), B, nh,
              nkv, page_size, int(window), float(scale), int(splits), _p(table),
              int(rot) if table is not None else 0, int(bool(write)), _stream()),
            "attn_decode_rope")
        return out
    f = _fn("attention_bf16", "gf_attn_decode",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
             c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p], defines,
            kernels=1)
    _ok(f(_p(qkv), qkv.stride(0), _p(pages[0]), _p(pages[1]), _p(block_table),
          block_table.stride(0), _p(cu_seqlens_q), _p(positions), _p(out), _p(scratch), B, nh,
          nkv, page_size, int(window), float(scale), int(splits), _stream()), "attn_decode")
    return out


def prefill(qkv, pages, block_table, cu_seqlens_q, kv_lens, B, max_q_len, nh, nkv, hd, scale,
            window, page_size, out=None):
    from . import _fn, _ok, _p, _stream
    if out is None:
        out = torch.empty((qkv.shape[0], nh * hd), dtype=torch.bfloat16, device=qkv.device)
    f = _fn("attention_bf16", "gf_attn_prefill",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p],
            (f"GF_HEAD_DIM={hd}",))
    _ok(f(_p(qkv), qkv.stride(0), _p(pages[0]), _p(pages[1]), _p(block_table),
          block_table.stride(0), _p(cu_seqlens_q), _p(kv_lens), _p(out), B, int(max_q_len), nh,
          nkv, page_size, int(window), float(scale), _stream()), "attn_prefill")
    return out


def tc_supports(hd: int, page_size: int) -> bool:
    return hd in (64, 128) and page_size % 8 == 0 and 128 % page_size == 0


# GINFER_B200_ATTN_POLY_EXP=n: every n-th exponential of an unmasked tile of the tcgen05 prefill
# kernel is computed by a polynomial on the FMA pipe instead of the special-function unit (0:
# none, which is also the default: no share measured faster).  A build of its own for each value.
POLY_EXP_EVERY = int(os.environ.get("GINFER_B200_ATTN_POLY_EXP") or 0)


def prefill_tc(qkv, pages, block_table, cu_seqlens_q, kv_lens, B, max_q_len, nh, nkv, hd, scale,
               window, page_size, trace=None, out=None, poly_exp_every: int | None = None):
    """Prefill attention on tcgen05 (``csrc/attention_tc.cu``); ``None`` if it cannot serve the
    shapes.  ``trace``: an int64 tensor of ``768 + 4 * CTAs`` slots that receives clock stamps of
    the first CTA's phases ([role 0 softmax (by tile), 1 MMA (by a stream's tile), 2 loader][32][8])
    and, behind them, every CTA's (start ns, end ns, SM) (for tuning; compiled into a build of its
    own).
    ``poly_exp_every``: see ``POLY_EXP_EVERY`` (``None``: that default)."""
    from ctypes import c_float, c_int, c_void_p

    from . import _fn, _ok, _p, _stream
    from .gemm_bf16 import _dev_state
    if not tc_supports(hd, page_size) or qkv.stride(0) % 8:
        return None
    T = qkv.shape[0]
    if out is None:
        out = torch.empty((T, nh * hd), dtype=torch.bfloat16, device=qkv.device)
    every = POLY_EXP_EVERY if poly_exp_every is None else int(poly_exp_every)
    defines = (f"GF_HEAD_DIM={hd}",) + ((f"GF_POLY_EXP_EVERY={every}",) if every > 0 else ())
    if trace is not None:
        defines += ("GF_TRACE",)          # a build of its own: the phase stamps cost the issuing thread time
    f = _fn("attention_tc", "gf_attn_prefill_tc",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
             c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
             c_void_p, c_void_p], defines)
    rc = f(_p(qkv), qkv.stride(0), _p(pages[0]), _p(pages[1]), pages.shape[1], _p(block_table),
           block_table.stride(0), _p(cu_seqlens_q), _p(kv_lens), _p(out), T, B, int(max_q_len),
           nh, nkv, page_size, int(window), float(scale), _p(_dev_state(qkv.device)["err"]),
           _p(trace), _stream())
    if rc == -6:
        return None
    _ok(rc, "attn_prefill_tc")
    return out


TC_MIN_QUERY_ROWS = 64      # below this a portion is too short to fill 128-row tiles


def fuses_rope(qkv, ctx, hd: int, nh: int, nkv: int) -> bool:
    """Whether attention over this step rotates q and k and writes the cache by itself (bf16
    decode steps), so that the caller skips the kernel that would do it before."""
    return qkv.dtype == torch.bfloat16 and ctx.decode_only and supports(hd, nh, nkv)


def try_run(qkv, pages, block_table, ctx, nh, nkv, hd, scale, window, page_size, rope=None):
    """Run a bf16 kernel if one takes this head size; ``None`` hands the work to the plain
    fp32-arithmetic kernel.  ``rope``: see :func:`decode` (only where :func:`fuses_rope`)."""
    if not supports(hd, nh, nkv):
        return None
    if ctx.decode_only:
        keys = ctx.max_kv_len if window <= 0 else min(window, ctx.max_kv_len)
        splits, parts = decode_partition(ctx.num_seqs, nh, nkv, keys)
        if ctx.extras.get("decode_splits"):
            splits, parts = ctx.extras["decode_splits"], 1
        if not tma_serves(hd, page_size, splits):
            parts = 1
        return decode(qkv, pages, block_table, ctx.cu_seqlens_q, ctx.positions, ctx.num_seqs, nh,
                      nkv, hd, scale, window, page_size, splits, rope=rope, parts=parts)
    assert rope is None, "only decode steps rotate inside the attention kernel"
    # A mixed step whose single tokens come first (as the scheduler orders them): those requests
    # go to the decode kernel, the portions behind them to a prefill kernel.  (A single token as a
    # portion of its own costs a whole tile of query rows per head.)
    B, nd = ctx.num_seqs, 0
    q_lens = ctx.q_lens_host
    while nd < B and nd < len(q_lens) and q_lens[nd] == 1:
        nd += 1
    out, cu, kv_lens, table, max_q = None, ctx.cu_seqlens_q, ctx.kv_lens, block_table, ctx.max_q_len
    if 0 < nd < B and len(q_lens) == B:
        keys = ctx.max_kv_len if window <= 0 else min(window, ctx.max_kv_len)
        out = torch.empty((qkv.shape[0], nh * hd), dtype=torch.bfloat16, device=qkv.device)
        splits, parts = decode_partition(nd, nh, nkv, keys)
        decode(qkv, pages, block_table[:nd], None, ctx.positions, nd, nh, nkv, hd, scale, window,
               page_size, splits, out=out, parts=parts if tma_serves(hd, page_size, splits) else 1)
        cu, kv_lens, table, B = cu[nd:], kv_lens[nd:], block_table[nd:], B - nd
        max_q = max(q_lens[nd:])
    if max_q >= TC_MIN_QUERY_ROWS:
        res = prefill_tc(qkv, pages, table, cu, kv_lens, B, max_q, nh, nkv, hd, scale, window,
                         page_size, out=out)
        if res is not None:
            return res
    return prefill(qkv, pages, table, cu, kv_lens, B, max_q, nh, nkv, hd, scale, window, page_size,
                   out=out)
