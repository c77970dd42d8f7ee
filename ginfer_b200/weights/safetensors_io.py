"""Reader and writer for the safetensors container.

Format, as the reference reads it (``ginfer/model/loader/safetensor_loader.cc:13-56``): an
unsigned 64-bit little-endian header length, a JSON header mapping tensor name to ``dtype``,
``shape`` and ``data_offsets`` (relative to the first byte after the header; the key
``__metadata__`` is skipped), then raw little-endian tensor bytes.  The byte range of a tensor is
checked against ``prod(shape) * sizeof(dtype)`` (``safetensor_loader.cc:70-74``).

The file is memory-mapped; a tensor is a zero-copy view of the mapping until it is cast or sent
to the device.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


_DTYPES: dict[str, tuple[torch.dtype, int]] = {
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "F64": (torch.float64, 8),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: tuple[int, ...]
    begin: int
    end: int


class SafetensorsFile:
    """One mapped ``.safetensors`` file."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"cannot open {path}: {e}") from e
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file ({size} bytes)")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._mm[:8])
        if 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file size {size}")
        try:
            header = json.loads(self._mm[8:8 + hlen].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from e
        self._base = 8 + hlen
        self.metadata = header.pop("__metadata__", {}) or {}
        self.entries: dict[str, TensorEntry] = {}
        for name, meta in header.items():
            code = meta.get("dtype")
            if code not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {code!r}")
            dt, esz = _DTYPES[code]
            shape = tuple(int(s) for s in meta["shape"])
            b, e = (int(x) for x in meta["data_offsets"])
            want = int(np.prod(shape, dtype=np.int64)) * esz if shape else esz
            if e - b != want:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' has {e - b} bytes but shape {list(shape)} of "
                    f"{code} needs {want}")
            if self._base + e > size:
                raise SafetensorsError(f"{path}: tensor '{name}' reaches past the end of the file")
            self.entries[name] = TensorEntry(name, dt, shape, b, e)
        self._buf = np.frombuffer(self._mm, dtype=np.uint8)

    def names(self) -> list[str]:
        return list(self.entries)

    def get(self, name: str) -> torch.Tensor:
        """A CPU tensor over the mapping (read-only memory: cast or copy before writing)."""
        ent = self.entries.get(name)
        if ent is None:
            raise SafetensorsError(f"{self.path}: tensor not found: {name}")
        raw = self._buf[self._base + ent.begin:self._base + ent.end]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")       # non-writable numpy buffer
            t = torch.from_numpy(raw)
        return t.view(ent.dtype).reshape(ent.shape)


def open_model_tensors(model_dir: str) -> dict[str, tuple[SafetensorsFile, str]]:
    """Map every tensor name of a model folder to (file, name).  Reads ``model.safetensors`` or,
    if present, ``model.safetensors.index.json`` and the shards it lists."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    out: dict[str, tuple[SafetensorsFile, str]] = {}
    if os.path.exists(index):
        with open(index, "r", encoding="utf-8") as f:
            weight_map = json.load(f)["weight_map"]
        files: dict[str, SafetensorsFile] = {}
        for name, fname in weight_map.items():
            if fname not in files:
                files[fname] = SafetensorsFile(os.path.join(model_dir, fname))
            out[name] = (files[fname], name)
        return out
    if not os.path.exists(single):
        raise SafetensorsError(f"no model.safetensors (or index) in {model_dir}")
    sf = SafetensorsFile(single)
    for name in sf.names():
        out[name] = (sf, name)
    return out


def write_safetensors(path: str, tensors: dict[str, torch.Tensor], metadata=None) -> None:
    """Write ``tensors`` (CPU, any of the supported dtypes) in name order."""
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} (tensor '{name}')")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [off, off + nbytes]}
        blobs.append(t)
        off += nbytes
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for t in blobs:
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)
