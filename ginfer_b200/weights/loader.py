"""Bind safetensors tensors to a model by name.

The reference binds by Hugging Face tensor name with no renaming (``ginfer/model/qwen2.cc:34-46``,
``ginfer/model/loader/model_loader.cc:56-76``) and fails on the first missing tensor
(``safetensor_loader.cc:62``).  Here the model says which tensors it needs
(:meth:`DecoderModel.tensor_specs`), and every problem of a folder (missing tensors, tensors
nobody asked for, wrong shapes) is reported in one error.

How a tensor is kept: matrices and embeddings in the compute dtype; biases and norm weights in the
compute dtype unless the file stores them in 32-bit, in which case they stay 32-bit; integer
tables as int32.  With ``float32`` as compute dtype every floating tensor becomes 32-bit.
"""
from __future__ import annotations

import re

import torch

from .safetensors_io import open_model_tensors


class WeightError(ValueError):
    """The tensors of a model folder do not fit the model."""

    def __init__(self, model_dir, missing, unexpected, wrong_shape, wrong_dtype=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = [f"weights in {model_dir} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n}: file has {list(got)}, model needs {list(want)}"
                for n, got, want in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong dtype ({len(self.wrong_dtype)}): " + ", ".join(
                f"{n}: {dt} cannot serve as {role}" for n, dt, role in self.wrong_dtype))
        super().__init__("\n".join(lines))


_FLOATS = (torch.float32, torch.float16, torch.bfloat16, torch.float64)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


def kept_dtype(role: str, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    """The dtype a tensor of ``role`` stored as ``stored`` has in memory."""
    if role == "int":
        return torch.int32
    if compute == torch.float32:
        return torch.float32
    if role in ("bias", "norm") and stored in (torch.float32, torch.float64):
        return torch.float32
    return compute


def check_and_convert(specs, available: dict, fetch, model_dir: str, compute: torch.dtype,
                      device, ignored=()) -> dict[str, torch.Tensor]:
    """``available``: name -> (shape, dtype) of what the folder holds; ``fetch(name)`` -> CPU
    tensor.  Returns name -> device tensor for every spec, or raises one :class:`WeightError`."""
    wanted = {s.name: s for s in specs}
    missing = [n for n in wanted if n not in available]
    pats = [re.compile(p) for p in ignored]
    unexpected = [n for n in available
                  if n not in wanted and not any(p.fullmatch(n) for p in pats)]
    wrong_shape, wrong_dtype = [], []
    for n, s in wanted.items():
        if n in available:
            shape, dt = available[n]
            if tuple(shape) != tuple(s.shape):
                wrong_shape.append((n, tuple(shape), tuple(s.shape)))
            if (s.role == "int") != (dt in _INTS) or (dt not in _FLOATS and dt not in _INTS):
                wrong_dtype.append((n, dt, s.role))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(model_dir, sorted(missing), sorted(unexpected), wrong_shape, wrong_dtype)
    out = {}
    up = Uploader(device) if torch.device(device).type == "cuda" else None
    for n, s in wanted.items():
        t = fetch(n)
        kept = kept_dtype(s.role, t.dtype, compute)
        if up is not None:
            out[n] = up.put(t, kept)
        else:
            out[n] = t.to(device=device, dtype=kept).contiguous()
    if up is not None:
        up.finish()
    return out


class Uploader:
    """Tensors of a file mapping to the device through two pinned staging buffers: the host copies
    the next piece out of the mapping while the device still receives the one before, and a
    tensor stored in another dtype than it is kept in is converted on the device.  The reference
    copies each tensor synchronously from pageable memory
    (``ginfer/core/tensor/tensor.cc:76-90``).  Each tensor keeps an allocation of its own (no
    slab): parts join tensors when they load (q|k|v, gate|up) and the originals are then freed."""

    def __init__(self, device, staging_bytes: int = 64 << 20):
        self.device = torch.device(device)
        self.size = int(staging_bytes)
        self.bufs = [torch.empty(self.size, dtype=torch.uint8, pin_memory=True) for _ in range(2)]
        self.free = [torch.cuda.Event(), torch.cuda.Event()]      # the buffer's copy has left it
        self.used = [False, False]
        self.turn = 0
        self.bytes = 0

    def put(self, t: torch.Tensor, kept: torch.dtype) -> torch.Tensor:
        """``t`` (CPU, contiguous) as a device tensor of dtype ``kept``."""
        t = t.contiguous()
        raw = t.reshape(-1).view(torch.uint8)
        with torch.cuda.device(self.device):
            dev = torch.empty(t.shape, dtype=t.dtype, device=self.device)
            dst = dev.reshape(-1).view(torch.uint8)
            for off in range(0, raw.numel(), self.size):
                n = min(self.size, raw.numel() - off)
                i = self.turn
                self.turn ^= 1
                if self.used[i]:
                    self.free[i].synchronize()
                self.bufs[i][:n].copy_(raw[off:off + n])          # out of the mapping
                dst[off:off + n].copy_(self.bufs[i][:n], non_blocking=True)
                self.free[i].record()
                self.used[i] = True
            self.bytes += raw.numel()
            return dev if kept == t.dtype else dev.to(kept)

    def finish(self) -> None:
        torch.cuda.synchronize(self.device)


def load_weights(model, model_dir: str, dtype: torch.dtype, device) -> None:
    """Read ``model_dir``'s safetensors into ``model`` (a :class:`DecoderModel`)."""
    index = open_model_tensors(model_dir)
    available = {n: (f.entries[k].shape, f.entries[k].dtype) for n, (f, k) in index.items()}
    tensors = check_and_convert(model.tensor_specs(), available,
                                lambda n: index[n][0].get(index[n][1]), model_dir, dtype,
                                device, ignored=getattr(model.plan, "ignored_tensors", ()))
    model.load(tensors, dtype, torch.device(device))
