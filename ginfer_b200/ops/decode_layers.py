"""All layers of a decode step in one persistent kernel (``csrc/decode_layers.cu``).

:class:`DecodeLayers` describes a stack of layers of one shape -- RMS norm, joined q/k/v product,
rotary encoding, paged attention, output product, RMS norm, gate/up product with SiLU, down
product -- by their weight tensors and cache bindings, and runs steps of at most 16 requests, one
token each, in bfloat16.  It knows nothing about models: a caller that recognises such a stack in
its plan hands the tensors over (``ginfer_b200/engine/fused_decode.py`` does that).
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_float, c_int, c_longlong, c_void_p
from dataclasses import dataclass

import torch

from .build import load_library


class NotServed(RuntimeError):
    """The kernel does not take this shape (the caller runs the layers one kernel at a time)."""


@dataclass
class LayerTensors:
    w_qkv: torch.Tensor            # [(heads + 2 kv heads) * head size, hidden] bf16
    w_out: torch.Tensor            # [hidden, heads * head size]
    w_gate_up: torch.Tensor        # [2 * intermediate, hidden], rows interleaved (gate_i, up_i)
    w_down: torch.Tensor           # [hidden, intermediate]
    b_qkv: torch.Tensor | None     # fp32
    b_out: torch.Tensor | None
    b_down: torch.Tensor | None
    gamma_mixer: torch.Tensor
    eps_mixer: float
    gamma_ff: torch.Tensor
    eps_ff: float


def _lib(head_dim: int):
    lib = load_library("decode_layers", (f"GF_HEAD_DIM={head_dim}",))
    if not getattr(lib, "_gf_typed", False):
        lib.gf_dl_create.restype = c_void_p
        lib.gf_dl_create.argtypes = [c_int] * 7 + [c_float, c_int, POINTER(c_int)]
        lib.gf_dl_destroy.restype = None
        lib.gf_dl_destroy.argtypes = [c_void_p]
        lib.gf_dl_sizes.restype = None
        lib.gf_dl_sizes.argtypes = [c_void_p, POINTER(c_longlong), POINTER(c_int)]
        lib.gf_dl_layer_bytes.restype = c_int
        lib.gf_dl_max_tokens.restype = c_int
        lib.gf_dl_set_layer.restype = c_int
        lib.gf_dl_set_layer.argtypes = [c_void_p, c_int] + [c_void_p] * 8 + \
            [c_int, c_float, c_void_p, c_int, c_float]
        lib.gf_dl_set_cache.restype = c_int
        lib.gf_dl_set_cache.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int]
        lib.gf_dl_upload.restype = c_int
        lib.gf_dl_upload.argtypes = [c_void_p, c_void_p, c_void_p]
        lib.gf_dl_run.restype = c_int
        lib.gf_dl_run.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                  POINTER(c_void_p), POINTER(c_int), c_int, POINTER(c_void_p),
                                  c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]
        lib._gf_typed = True
    return lib


def _ptr(t):
    if t is not None and not t.is_cuda:
        raise RuntimeError("ginfer_b200 kernels run on a CUDA device only; got a tensor on "
                           f"{t.device}")
    return None if t is None else c_void_p(t.data_ptr())


class DecodeLayers:
    MAX_TOKENS = 16

    def __init__(self, num_layers: int, hidden: int, heads: int, kv_heads: int, head_dim: int,
                 intermediate: int, page_size: int, rot: int, scale: float, device):
        if head_dim % 16 or not 16 <= head_dim <= 256:
            raise NotServed(f"head size {head_dim}")
        self.device = torch.device(device)
        self.lib = _lib(head_dim)
        status = c_int(0)
        with torch.cuda.device(self.device):
            self.handle = self.lib.gf_dl_create(num_layers, hidden, heads, kv_heads, intermediate,
                                                page_size, rot, scale, self.device.index or 0,
                                                ctypes.byref(status))
        if not self.handle:
            raise NotServed({1: "sizes", 2: "shared memory", 3: "device"}.get(status.value, "?"))
        self.num_layers, self.hidden, self.heads, self.kv_heads = num_layers, hidden, heads, kv_heads
        self.head_dim, self.intermediate = head_dim, intermediate
        sizes = (c_longlong * 9)()
        sched = (c_int * 8)()
        self.lib.gf_dl_sizes(self.handle, sizes, sched)
        self.schedule = {"splits": list(sched[:4]), "stages": sched[4], "ctas": sched[5],
                         "shared_bytes": sched[6]}
        dts = [torch.float32] * 4 + [torch.bfloat16, torch.float32, torch.bfloat16, torch.int32,
               torch.bfloat16]
        self.bufs = [torch.zeros(int(n), dtype=dt, device=self.device)
                     for n, dt in zip(sizes, dts)]
        self.h = self.bufs[0].view(self.MAX_TOKENS, hidden)
        self._buf_ptrs = (c_void_p * 9)(*[b.data_ptr() for b in self.bufs])
        self.bar = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.layers_dev = torch.zeros(num_layers * self.lib.gf_dl_layer_bytes(), dtype=torch.uint8,
                                      device=self.device)
        self.stamps: torch.Tensor | None = None    # int64 [CTAs, 64]: set to time the first phases
        self._keep: list = []            # tensors whose addresses the descriptions hold
        self._uploaded = False

    def __del__(self):
        h, self.handle = getattr(self, "handle", None), None
        if h:
            self.lib.gf_dl_destroy(h)

    # ------------------------------------------------------------------ description
    def set_layer(self, i: int, t: LayerTensors) -> None:
        H, nh, nkv, hd, I = self.hidden, self.heads, self.kv_heads, self.head_dim, self.intermediate
        want = {"w_qkv": ((nh + 2 * nkv) * hd, H), "w_out": (H, nh * hd), "w_gate_up": (2 * I, H),
                "w_down": (H, I)}
        for name, shape in want.items():
            w = getattr(t, name)
            if tuple(w.shape) != shape or w.dtype != torch.bfloat16 or not w.is_contiguous() \
                    or w.data_ptr() % 16:
                raise NotServed(f"{name}: {tuple(w.shape)} {w.dtype}, wanted bf16 {shape}")
        for b in (t.b_qkv, t.b_out, t.b_down):
            if b is not None and (b.dtype != torch.float32 or not b.is_contiguous()):
                raise NotServed("biases are kept in fp32")
        for g in (t.gamma_mixer, t.gamma_ff):
            if g.dtype not in (torch.bfloat16, torch.float32) or g.numel() != H \
                    or g.data_ptr() % 16:
                raise NotServed("norm weights")
        rc = self.lib.gf_dl_set_layer(
            self.handle, i, _ptr(t.w_qkv), _ptr(t.w_out), _ptr(t.w_gate_up), _ptr(t.w_down),
            _ptr(t.b_qkv), _ptr(t.b_out), _ptr(t.b_down), _ptr(t.gamma_mixer),
            int(t.gamma_mixer.dtype == torch.float32), float(t.eps_mixer), _ptr(t.gamma_ff),
            int(t.gamma_ff.dtype == torch.float32), float(t.eps_ff))
        if rc:
            raise NotServed(f"layer {i}: tensor maps could not be made (code {rc})")
        self._keep.append(t)
        self._uploaded = False

    MAX_GROUPS = 4

    def set_cache(self, i: int, kpages: torch.Tensor, vpages: torch.Tensor, group: int,
                  window: int, write: bool) -> None:
        """Layer ``i`` keeps its keys and values in ``kpages`` / ``vpages``
        ``[pages, page, kv heads, head size]`` and finds them by block table ``group``."""
        assert kpages.dtype == torch.bfloat16 and kpages.is_contiguous() and vpages.is_contiguous()
        rc = self.lib.gf_dl_set_cache(self.handle, i, _ptr(kpages), _ptr(vpages), int(group),
                                      int(window), int(bool(write)))
        if rc:
            raise NotServed(f"cache group {group}")
        self._keep.append((kpages, vpages))
        self._uploaded = False

    def upload(self) -> None:
        stream = c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        rc = self.lib.gf_dl_upload(self.handle, _ptr(self.layers_dev), stream)
        if rc:
            raise RuntimeError(f"decode_layers: CUDA error {rc} while copying the descriptions")
        self._uploaded = True

    # ------------------------------------------------------------------ a step
    def run(self, num_tokens: int, positions: torch.Tensor, rope: torch.Tensor | None,
            block_tables: list[torch.Tensor], token_ids: torch.Tensor | None = None,
            embedding: torch.Tensor | None = None,
            stop: tuple[int, int] = (-1, -1)) -> torch.Tensor:
        """Run the layers for ``num_tokens`` requests.  The residual stream starts as the
        embedding rows of ``token_ids`` (or as what ``self.h`` holds) and is returned:
        ``[num_tokens, hidden]`` fp32, a view of ``self.h``.  ``block_tables[g]``: int32
        ``[requests, width]`` of cache group ``g``, rows in the order of the tokens."""
        from . import _Counter
        if not self._uploaded:
            self.upload()
        stream = c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        _Counter.launches += 1
        n = len(block_tables)
        tables = (c_void_p * n)(*[t.data_ptr() for t in block_tables])
        strides = (c_int * n)(*[t.stride(0) for t in block_tables])
        rc = self.lib.gf_dl_run(self.handle, num_tokens, _ptr(token_ids), _ptr(embedding),
                                _ptr(positions), _ptr(rope), tables, strides, n,
                                self._buf_ptrs, _ptr(self.bar),
                                _ptr(self.err), stop[0], stop[1], _ptr(self.stamps), stream)
        if rc:
            raise RuntimeError(f"decode_layers: launch failed (code {rc})")
        return self.h[:num_tokens]

    def check_errors(self) -> None:
        code = int(self.err.item())
        if code:
            self.err.zero_()
            raise RuntimeError(f"decode_layers: a wait inside the kernel ran out (code {code})")
