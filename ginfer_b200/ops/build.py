"""Compile the CUDA sources under ``csrc/`` for sm_100a and load them through ``ctypes``.

Every ``.cu`` file becomes one shared library with a C interface (raw device pointers, sizes and a
stream).  A library is compiled the first time something needs it, into ``csrc/_build/`` inside
the package (or ``$GINFER_B200_BUILD_DIR``, or a per-user folder under the system's temporary
folder when the package is read-only); its file name carries a hash of the sources and flags, so a
changed source is compiled again and an unchanged one is found.  There is no fall-back: a missing
compiler or a failed compilation raises.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

CSRC_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-lineinfo", "-std=c++17", "--shared", "-Xcompiler", "-fPIC"]

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()
_dir_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("GINFER_B200_NVCC"), shutil.which("nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc was not found (set GINFER_B200_NVCC or put it on PATH); the CUDA "
                     "kernels of ginfer_b200 cannot be built and there is no other code path")


def _writable(d: str) -> bool:
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".probe-{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


_build_dir_cache: str | None = None


def build_dir() -> str:
    global _build_dir_cache
    with _dir_lock:
        return _build_dir_locked()


def _build_dir_locked() -> str:
    global _build_dir_cache
    if _build_dir_cache:
        return _build_dir_cache
    cands = []
    if os.environ.get("GINFER_B200_BUILD_DIR"):
        cands.append(os.environ["GINFER_B200_BUILD_DIR"])
    cands.append(os.path.join(CSRC_DIR, "_build"))
    cands.append(os.path.join(tempfile.gettempdir(), f"ginfer_b200_build_{os.getuid()}"))
    for d in cands:
        if _writable(d):
            _build_dir_cache = d
            return d
    raise BuildError(f"no writable build folder among {cands}")


def _headers() -> list[str]:
    return sorted(os.path.join(CSRC_DIR, f) for f in os.listdir(CSRC_DIR)
                  if f.endswith((".cuh", ".h")))


def _digest(source: str, defines: tuple[str, ...]) -> str:
    h = hashlib.sha256()
    for path in [source] + _headers():
        with open(path, "rb") as f:
            h.update(os.path.basename(path).encode() + b"\0" + f.read())
    h.update(" ".join(ARCH_FLAGS + BASE_FLAGS + list(defines)).encode())
    return h.hexdigest()[:16]


def library_path(name: str, defines: tuple[str, ...] = ()) -> tuple[str, str]:
    source = os.path.join(CSRC_DIR, name + ".cu")
    if not os.path.exists(source):
        raise BuildError(f"no CUDA source {source}")
    tag = "".join(f"_{d.replace('=', '')}" for d in defines)
    return source, os.path.join(build_dir(), f"gf_{name}{tag}-{_digest(source, defines)}.so")


def compile_library(name: str, defines: tuple[str, ...] = (), verbose: bool = True) -> str:
    """Compile ``csrc/<name>.cu`` with ``-D`` for each of ``defines`` unless it is built
    already; return the path of the shared library."""
    source, so = library_path(name, defines)
    if os.path.exists(so):
        return so
    tmp = f"{so}.{os.getpid()}.tmp"
    cmd = [_nvcc()] + ARCH_FLAGS + BASE_FLAGS + [f"-D{d}" for d in defines] + \
          ["-I", CSRC_DIR, "-o", tmp, source]
    if verbose:
        print(f"[ginfer_b200] compiling {os.path.basename(source)}"
              f"{' ' + ' '.join(defines) if defines else ''} for sm_100a ...",
              file=sys.stderr, flush=True)
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    last = t0
    while True:
        try:
            out, _ = proc.communicate(timeout=5)
            break
        except subprocess.TimeoutExpired:
            if verbose and time.time() - last >= 15:
                last = time.time()
                print(f"[ginfer_b200]   ... still compiling {name} ({int(last - t0)} s)",
                      file=sys.stderr, flush=True)
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise BuildError(f"nvcc failed on {source} (exit {proc.returncode}):\n{out}")
    os.replace(tmp, so)
    if verbose:
        print(f"[ginfer_b200]   built {os.path.basename(so)} in {time.time() - t0:.1f} s",
              file=sys.stderr, flush=True)
    return so


_pdl_enabled = os.environ.get("GINFER_B200_PDL", "1") != "0"


def load_library(name: str, defines: tuple[str, ...] = ()) -> ctypes.CDLL:
    key = name + "|" + "|".join(defines)
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            lib = ctypes.CDLL(compile_library(name, defines))
            if hasattr(lib, "gf_set_pdl"):
                lib.gf_set_pdl(ctypes.c_int(1 if _pdl_enabled else 0))
            _loaded[key] = lib
        return lib


def set_pdl(enabled: bool) -> None:
    """Switch programmatic dependent launch on or off for every kernel library (those loaded and
    those yet to be).  On by default; ``GINFER_B200_PDL=0`` in the environment turns it off."""
    global _pdl_enabled
    with _lock:
        _pdl_enabled = bool(enabled)
        for lib in _loaded.values():
            if hasattr(lib, "gf_set_pdl"):
                lib.gf_set_pdl(ctypes.c_int(1 if _pdl_enabled else 0))


# sources that are compiled per head size but take only some head sizes (the tcgen05 attention)
HEAD_DIMS_OF = {"attention_tc": (64, 128)}


# every library the framework can ask for: (source name, defines)
def all_libraries(head_dims=(64, 128)) -> list[tuple[str, tuple[str, ...]]]:
    libs: list[tuple[str, tuple[str, ...]]] = []
    for f in sorted(os.listdir(CSRC_DIR)):
        if not f.endswith(".cu"):
            continue
        name = f[:-3]
        with open(os.path.join(CSRC_DIR, f), "r", encoding="utf-8") as fh:
            per_head_dim = "GF_HEAD_DIM" in fh.read()
        if per_head_dim:
            only = HEAD_DIMS_OF.get(name)
            libs += [(name, (f"GF_HEAD_DIM={hd}",)) for hd in head_dims
                     if only is None or hd in only]
        else:
            libs.append((name, ()))
    return libs


def build_all(head_dims=(64, 128), verbose: bool = True) -> list[str]:
    """Compile everything (in parallel); used by the build check."""
    from concurrent.futures import ThreadPoolExecutor
    libs = all_libraries(head_dims)
    with ThreadPoolExecutor(max_workers=min(8, len(libs) or 1)) as ex:
        return list(ex.map(lambda nd: compile_library(nd[0], nd[1], verbose), libs))
