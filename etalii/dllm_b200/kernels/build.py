"""Compiles the CUDA sources of `csrc/` for sm_100a with nvcc and loads them with ctypes.

Each source file becomes one shared library, built the first time one of its kernels is needed and kept beside the
sources under `csrc/_build/` (named by a hash of the sources and flags, so an edit rebuilds). There is no fallback:
a missing compiler, a failed build or a library that does not load raises `KernelBuildError`.
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

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

SOURCES = {
    "elementwise": "elementwise.cu",
    "gemm_simt": "gemm_simt.cu",
    "gemm_bf16": "gemm_bf16.cu",
    "gemv": "gemv.cu",
    "gemv_tma": "gemv_tma.cu",
    "gemv_cluster": "gemv_cluster.cu",
    "mlp_decode": "mlp_decode.cu",
    "gemm_tcgen05": "gemm_tcgen05.cu",
    "attention": "attention.cu",
    "attention_decode": "attention_decode.cu",
    "attention_decode_cluster": "attention_decode_cluster.cu",
    "attention_prefill": "attention_prefill.cu",
    "attention_prefill_tcgen05": "attention_prefill_tcgen05.cu",
    "attention_decode_static": "attention_decode_static.cu",
    "sampling": "sampling.cu",
    "step_launcher": "step_launcher.cu",
}
"""Library name -> source file. A library added here is built by `build_all` and loadable by `library`."""

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class KernelBuildError(RuntimeError):
    pass


def _nvcc() -> str:
    found = shutil.which("nvcc")
    for candidate in (found, "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.isfile(candidate):
            return candidate
    raise KernelBuildError("nvcc was not found: the sm_100a kernels cannot be built (there is no fallback path)")


_build_dir_found: str | None = None
_build_dir_lock = threading.Lock()


def _build_dir() -> str:
    """Where libraries are kept: found once (libraries may be built from several threads at a time)."""
    global _build_dir_found
    with _build_dir_lock:
        if _build_dir_found is not None and os.path.isdir(_build_dir_found):
            return _build_dir_found
        override = os.environ.get("DLLM_B200_BUILD_DIR")
        candidates = [override] if override else []
        candidates.append(os.path.join(CSRC, "_build"))
        candidates.append(os.path.join(tempfile.gettempdir(), f"dllm_b200_build_{os.getuid()}"))
        for path in candidates:
            try:
                os.makedirs(path, exist_ok=True)
                probe = os.path.join(path, f".write_{os.getpid()}_{threading.get_ident()}")
                with open(probe, "w"):
                    pass
                os.remove(probe)
                _build_dir_found = path
                return path
            except OSError:
                continue
        raise KernelBuildError(f"no writable build directory among {candidates}")


def _digest(source: str) -> str:
    sha = hashlib.sha256()
    sha.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    headers = sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))
    included = []  # other sources this one includes as text
    with open(os.path.join(CSRC, source), encoding="utf-8") as handle:
        for line in handle:
            line = line.strip()
            if line.startswith("#include \"") and line.endswith(".cu\""):
                included.append(line.split("\"")[1])
    for name in [source, *included, *headers]:
        with open(os.path.join(CSRC, name), "rb") as handle:
            sha.update(name.encode())
            sha.update(handle.read())
    return sha.hexdigest()[:16]


def library_path(name: str) -> str:
    source = SOURCES[name]
    return os.path.join(_build_dir(), f"libdllm_b200_{name}-{_digest(source)}.so")


def _run_nvcc(source: str, path: str, flags, verbose: bool) -> None:
    """Compiles `source` into the shared library `path` (written under a temporary name first), printing a line now
    and then while nvcc runs."""
    label = os.path.basename(source)
    temporary = f"{path}.{os.getpid()}.tmp"
    command = [_nvcc(), *ARCH_FLAGS, *NVCC_FLAGS, *flags, "-I", CSRC, source, "-o", temporary]
    if verbose:
        print(f"[dllm_b200] compiling {label} for sm_100a ...", file=sys.stderr, flush=True)
    start = time.time()
    process = subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            output, _ = process.communicate(timeout=10)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[dllm_b200] ... still compiling {label} ({time.time() - start:.0f} s)",
                      file=sys.stderr, flush=True)
    if process.returncode != 0:
        if os.path.exists(temporary):
            os.remove(temporary)
        raise KernelBuildError(f"nvcc failed on {label}:\n{output}")
    os.replace(temporary, path)
    if verbose:
        print(f"[dllm_b200] built {os.path.basename(path)} in {time.time() - start:.1f} s", file=sys.stderr, flush=True)


def compile_library(name: str, verbose: bool = True) -> str:
    """Builds the library if its file is not there yet; returns the path."""
    path = library_path(name)
    if os.path.isfile(path):
        return path
    _run_nvcc(os.path.join(CSRC, SOURCES[name]), path, (), verbose)
    prefix = f"libdllm_b200_{name}-"
    for stale in os.listdir(os.path.dirname(path)):  # older builds of the same source
        if stale.startswith(prefix) and stale.endswith(".so") and stale != os.path.basename(path):
            try:
                os.remove(os.path.join(os.path.dirname(path), stale))
            except OSError:
                pass
    return path


def compile_extra(source: str, flags=(), verbose: bool = True) -> ctypes.CDLL:
    """Builds and loads a CUDA source that is not part of the library (a test's own kernel, a user's part) with the
    library's compiler flags plus `flags` and `csrc/` on the include path, so it can use the library's headers."""
    with open(source, "rb") as handle:
        sha = hashlib.sha256(handle.read())
    sha.update(" ".join([*ARCH_FLAGS, *NVCC_FLAGS, *flags]).encode())
    for name in sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))):
        with open(os.path.join(CSRC, name), "rb") as handle:
            sha.update(handle.read())
    stem = os.path.splitext(os.path.basename(source))[0]
    path = os.path.join(_build_dir(), f"libextra_{stem}-{sha.hexdigest()[:16]}.so")
    with _lock:
        if not os.path.isfile(path):
            _run_nvcc(source, path, tuple(flags), verbose)
        try:
            return ctypes.CDLL(path)
        except OSError as error:
            raise KernelBuildError(f"{path} does not load: {error}") from error


def library(name: str) -> ctypes.CDLL:
    """The loaded library `name`, compiled first if needed."""
    with _lock:
        if name not in _loaded:
            if name not in SOURCES:
                raise KernelBuildError(f"no kernel library named {name!r}")
            path = compile_library(name)
            try:
                _loaded[name] = ctypes.CDLL(path)
            except OSError as error:
                raise KernelBuildError(f"{path} does not load: {error}") from error
        return _loaded[name]


def prebuild(names, verbose: bool = True) -> None:
    """Compiles the named libraries that are not built yet, side by side (a model knows which ones its parts use;
    building them together at load time takes as long as the slowest, not as their sum)."""
    from concurrent.futures import ThreadPoolExecutor

    missing = [n for n in dict.fromkeys(names) if n in SOURCES and n not in _loaded and
               not os.path.isfile(library_path(n))]
    if len(missing) <= 1:
        for name in missing:
            compile_library(name, verbose)
        return
    with ThreadPoolExecutor(max_workers=min(len(missing), os.cpu_count() or 1)) as pool:
        list(pool.map(lambda name: compile_library(name, verbose), missing))


def build_all(verbose: bool = True, jobs: int | None = None) -> list[str]:
    """Builds every library (those that are missing), several nvcc processes at a time; returns the paths."""
    from concurrent.futures import ThreadPoolExecutor

    workers = max(1, min(jobs or (os.cpu_count() or 1), len(SOURCES)))
    with ThreadPoolExecutor(max_workers=workers) as pool:
        return list(pool.map(lambda name: compile_library(name, verbose), SOURCES))
