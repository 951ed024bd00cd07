"""Compiles the CUDA sources of this folder for sm_100a and loads them.

Each library is one `.cu` file compiled by `nvcc` into a shared object whose name carries
a hash of the source, the shared header and the flags, so a changed source is never
served by an old binary.  Binaries are kept in `_build/` beside the sources; if that
folder cannot be written they go to a folder under the system's temporary directory.
Nothing is compiled until a library is first asked for; a model therefore compiles what
it uses (an attention library, for instance, is specialised to one head size and dtype).
While the compiler runs a line is printed every few seconds.
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
from typing import Dict, Sequence

_HERE = os.path.dirname(os.path.abspath(__file__))
_ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
_BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-shared",
               "--expt-relaxed-constexpr", "-Xcompiler", "-fvisibility=hidden"]
_HEADERS = tuple(sorted(name for name in os.listdir(_HERE) if name.endswith((".cuh", ".h"))))
_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class ExtensionMissing(RuntimeError):
    """The CUDA extension cannot be built or loaded; nothing stands in for it."""


def _nvcc() -> str:
    for candidate in (os.environ.get("TAU_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.isfile(candidate):
            return candidate
    raise ExtensionMissing("nvcc was not found (looked at $TAU_NVCC, PATH and /usr/local/cuda/bin)")


def _build_dir() -> str:
    preferred = os.path.join(_HERE, "_build")
    try:
        os.makedirs(preferred, exist_ok=True)
        probe = os.path.join(preferred, f".probe-{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return preferred
    except OSError:
        fallback = os.path.join(tempfile.gettempdir(), f"tau_rs_b200_build_{os.getuid()}")
        os.makedirs(fallback, exist_ok=True)
        return fallback


def _flags(defines: Sequence[str]) -> list:
    return _ARCH_FLAGS + _BASE_FLAGS + [f"-D{define}" for define in defines]


def library_path(source: str, defines: Sequence[str] = ()) -> str:
    digest = hashlib.sha256()
    for name in (source, *_HEADERS):
        with open(os.path.join(_HERE, name), "rb") as handle:
            digest.update(handle.read())
    digest.update(" ".join(_flags(defines)).encode())
    stem = os.path.splitext(source)[0]
    tag = "".join(ch if ch.isalnum() else "_" for ch in "_".join(defines))
    name = f"{stem}{'_' + tag if tag else ''}_{digest.hexdigest()[:12]}.so"
    for folder in (os.path.join(_HERE, "_build"), os.path.join(tempfile.gettempdir(), f"tau_rs_b200_build_{os.getuid()}")):
        if os.path.isfile(os.path.join(folder, name)):
            return os.path.join(folder, name)
    return os.path.join(_build_dir(), name)


def compile_library(source: str, defines: Sequence[str] = (), verbose: bool = True) -> str:
    """Compiles `source` unless its binary exists; returns the binary's path."""
    target = library_path(source, defines)
    if os.path.isfile(target):
        return target
    command = [_nvcc(), *_flags(defines), "-o", target + f".tmp{os.getpid()}", os.path.join(_HERE, source)]
    label = source + (" [" + " ".join(defines) + "]" if defines else "")
    if verbose:
        print(f"[tau_rs_b200] compiling {label} for sm_100a ...", file=sys.stderr, flush=True)
    started = time.time()
    process = subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            output, _ = process.communicate(timeout=10)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[tau_rs_b200] still compiling {label} ({time.time() - started:.0f} s)", file=sys.stderr, flush=True)
    if process.returncode != 0:
        raise ExtensionMissing(f"nvcc failed on {source}:\n{output}")
    os.replace(target + f".tmp{os.getpid()}", target)
    if verbose:
        print(f"[tau_rs_b200] compiled {label} in {time.time() - started:.0f} s", file=sys.stderr, flush=True)
    return target


def load_library(source: str, defines: Sequence[str] = ()) -> ctypes.CDLL:
    key = source + "|" + "|".join(defines)
    with _lock:
        library = _loaded.get(key)
        if library is None:
            import torch  # the CUDA runtime's context is torch's

            path = compile_library(source, defines)
            try:
                library = ctypes.CDLL(path)
            except OSError as error:
                raise ExtensionMissing(f"cannot load {path}: {error}") from error
            _loaded[key] = library
        return library
