"""Compiles the CUDA sources under ``csrc/`` for sm_100a with nvcc and loads them.

Each ``.cu`` file becomes one shared library of ``extern "C"`` launchers, loaded with
ctypes.  A library is built at its first use (so a run compiles only what its model and
precision need), cached under a name that carries a hash of its sources and flags, and
printed about while it compiles.  There is no fallback: if nvcc is missing or fails, the
call raises ``KernelBuildError``.

The reference builds its CUDA file in ``build.rs`` (build.rs:143-228) for sm_61..sm_90;
here the only target is sm_100a.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import re
import shutil
import subprocess
import sys
import tempfile
import threading
import time

CSRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr", "-Wno-deprecated-gpu-targets"]

# library name -> (source file, extra nvcc flags)
LIBRARIES = {
    "ops": ("ops.cu", []),
    "gemm_simt": ("gemm_simt.cu", []),
    "attention": ("attention.cu", []),
    "sampling": ("sampling.cu", []),
    "gemm_tc": ("gemm_tc.cu", []),
    "attention_prefill": ("attention_prefill.cu", []),
    "attention_prefill_tc": ("attention_prefill_tc.cu", []),
}


class KernelBuildError(RuntimeError):
    pass


_lock = threading.Lock()
_loaded: dict[str, ctypes.CDLL] = {}


def _nvcc() -> str:
    for cand in (os.environ.get("MINFER_B200_NVCC"), shutil.which("nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise KernelBuildError(
        "nvcc was not found (looked at $MINFER_B200_NVCC, PATH and /usr/local/cuda/bin); "
        "the CUDA kernels cannot be built and there is no other path")


_build_dir_lock = threading.Lock()
_build_dir_found: list = []


def _build_dir() -> str:
    """In-tree ``minfer_b200/_lib`` when writable, else a per-user folder under the temp dir.
    Decided once per process (threads that compile side by side must agree on it)."""
    with _build_dir_lock:
        if not _build_dir_found:
            _build_dir_found.append(_find_build_dir())
        return _build_dir_found[0]


def _find_build_dir() -> str:
    env = os.environ.get("MINFER_B200_BUILD_DIR")
    candidates = [env] if env else []
    candidates.append(os.path.join(os.path.dirname(CSRC), "_lib"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"minfer_b200_lib_{os.getuid()}"))
    for c in candidates:
        try:
            os.makedirs(c, exist_ok=True)
            probe = os.path.join(c, f".probe_{os.getpid()}")
            with open(probe, "w") as f:
                f.write("")
            os.remove(probe)
            return c
        except OSError:
            continue
    raise KernelBuildError("no writable folder for the compiled kernels: tried " + ", ".join(candidates))


def _source_hash(source: str, flags: list[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(ARCH_FLAGS + BASE_FLAGS + flags).encode())
    for name in sorted(os.listdir(CSRC)):
        if name == source or name.endswith((".cuh", ".h")):
            with open(os.path.join(CSRC, name), "rb") as f:
                h.update(name.encode())
                h.update(f.read())
    return h.hexdigest()[:16]


def library_path(name: str) -> str:
    source, flags = LIBRARIES[name]
    return os.path.join(_build_dir(), f"libmf_{name}_{_source_hash(source, flags)}.so")


def remove_old_versions(name: str, keep: str) -> None:
    """Older builds of library ``name`` (other source hashes) beside ``keep`` are of no use any
    more.  The whole file name is matched: "attention" must not take "attention_prefill_tc"
    for its own."""
    own = re.compile(rf"libmf_{re.escape(name)}_[0-9a-f]{{16}}\.so")
    folder = os.path.dirname(keep)
    for other in os.listdir(folder):
        if own.fullmatch(other) and other != os.path.basename(keep):
            try:
                os.remove(os.path.join(folder, other))
            except OSError:
                pass


def compile_library(name: str, verbose: bool = True) -> str:
    """Builds the library if its file is not there yet; returns the path."""
    source, flags = LIBRARIES[name]
    out = library_path(name)
    if os.path.exists(out):
        return out
    nvcc = _nvcc()
    tmp = f"{out}.{os.getpid()}.tmp"
    cmd = [nvcc] + ARCH_FLAGS + BASE_FLAGS + flags + ["-I", CSRC, "-o", tmp,
                                                      os.path.join(CSRC, source)]
    if verbose:
        print(f"[minfer_b200] compiling {source} for sm_100a ...", file=sys.stderr, flush=True)
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            log, _ = proc.communicate(timeout=15)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[minfer_b200]   still compiling {source} ({time.time() - t0:.0f} s)",
                      file=sys.stderr, flush=True)
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise KernelBuildError(f"nvcc failed for {source}:\n{' '.join(cmd)}\n{log}")
    os.replace(tmp, out)
    remove_old_versions(name, out)
    if verbose:
        print(f"[minfer_b200] built {os.path.basename(out)} in {time.time() - t0:.1f} s",
              file=sys.stderr, flush=True)
    return out


def load_library(name: str) -> ctypes.CDLL:
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            lib = ctypes.CDLL(compile_library(name))
            _loaded[name] = lib
        return lib


def prebuild(names, verbose: bool = True) -> list[str]:
    """Compiles those of the named libraries that are not built yet, side by side (nvcc runs
    as a process of its own, a few seconds each); returns their paths."""
    names = [n for n in dict.fromkeys(names)]
    missing = [n for n in names if not os.path.exists(library_path(n))]
    if len(missing) > 1:
        from concurrent.futures import ThreadPoolExecutor
        with ThreadPoolExecutor(max_workers=min(len(missing), max(1, os.cpu_count() or 1))) as pool:
            list(pool.map(lambda n: compile_library(n, verbose), missing))
    return [compile_library(n, verbose) for n in names]


def build_all(verbose: bool = True) -> list[str]:
    """Compiles every library (cross-compiles without a GPU)."""
    return prebuild(list(LIBRARIES), verbose)
