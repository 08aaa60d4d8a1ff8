"""Builds and loads the package's native libraries.

Each library is a few source files compiled for sm_100a into one shared
object under `cellm_b200/_build/` (or, when the package folder cannot be
written, under the system's temporary folder). A library is compiled the
first time something asks for it and is found again by a hash of its sources
and flags, so a changed source is never served by a stale binary. The kernels
export plain C symbols and are called through ctypes; nothing here includes
torch's headers, which keeps a first build to seconds per file.
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

_HERE = os.path.dirname(os.path.abspath(__file__))
_PKG = os.path.dirname(_HERE)

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-Wall"]

# library name -> (compiler, sources relative to csrc/, extra flags)
LIBRARIES: dict[str, tuple[str, list[str], list[str]]] = {
    "runtime": ("c++", ["runtime/block_allocator.cc", "runtime/cache_manager.cc",
                        "runtime/scheduler.cc", "runtime/executor.cc", "runtime/c_api.cc"], []),
    "kernels_common": ("nvcc", ["kernels/embed.cu", "kernels/add_rmsnorm.cu", "kernels/short_conv.cu",
                                "kernels/qk_norm_rope.cu", "kernels/swiglu.cu", "kernels/sample.cu",
                                "kernels/attention_plain.cu"], []),
    "gemm_plain": ("nvcc", ["kernels/gemm_plain.cu"], []),
    "gemm_tcgen05": ("nvcc", ["kernels/gemm_tcgen05.cu"], []),
    "attention_flash": ("nvcc", ["kernels/attention_flash.cu"], []),
    "attention_decode": ("nvcc", ["kernels/attention_decode.cu"], []),
    "attention_tc": ("nvcc", ["kernels/attention_tc.cu"], []),
}

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[cellm_b200] {msg}", file=sys.stderr, flush=True)


def _find(tool: str, fallbacks: list[str]) -> str:
    p = shutil.which(tool)
    if p:
        return p
    for f in fallbacks:
        if os.path.isfile(f):
            return f
    raise BuildError(f"{tool} not found (looked on PATH and in {fallbacks})")


def nvcc_path() -> str:
    return _find("nvcc", ["/usr/local/cuda/bin/nvcc"])


def build_dir() -> str:
    """In-tree build folder if it can be written, else a per-user temporary one."""
    d = os.path.join(_PKG, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.unlink(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"cellm_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _key(compiler: str, sources: list[str], flags: list[str]) -> str:
    h = hashlib.sha256()
    h.update(compiler.encode())
    h.update(" ".join(flags).encode())
    seen = set()
    for s in sources:
        path = os.path.join(_HERE, s)
        with open(path, "rb") as f:
            h.update(f.read())
        # headers next to the sources take part in the key
        folder = os.path.dirname(path)
        if folder not in seen:
            seen.add(folder)
            for name in sorted(os.listdir(folder)):
                if name.endswith((".h", ".cuh", ".hpp")):
                    with open(os.path.join(folder, name), "rb") as f:
                        h.update(name.encode())
                        h.update(f.read())
    return h.hexdigest()[:16]


def library_path(name: str) -> str:
    compiler, sources, extra = LIBRARIES[name]
    flags = (NVCC_FLAGS if compiler == "nvcc" else CXX_FLAGS) + extra
    return os.path.join(build_dir(), f"lib{name}-{_key(compiler, sources, flags)}.so")


def _run(cmd: list[str], what: str) -> None:
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                            env={**os.environ, "HOME": os.environ.get("HOME") or tempfile.gettempdir()})
    t0 = time.time()
    out: list[str] = []
    reader = threading.Thread(target=lambda: out.append(proc.stdout.read()), daemon=True)
    reader.start()
    while True:
        try:
            proc.wait(timeout=10)
            break
        except subprocess.TimeoutExpired:
            _say(f"still compiling {what} ({time.time() - t0:.0f} s)")
    reader.join()
    if proc.returncode != 0:
        raise BuildError(f"compiling {what} failed ({proc.returncode}):\n{' '.join(cmd)}\n{''.join(out)}")


def build(name: str, force: bool = False) -> str:
    """Compile library `name` if its binary is missing; return the path."""
    compiler, sources, extra = LIBRARIES[name]
    path = library_path(name)
    if os.path.isfile(path) and not force:
        return path
    srcs = [os.path.join(_HERE, s) for s in sources]
    tmp = f"{path}.{os.getpid()}.tmp"
    _say(f"compiling {name} ({len(srcs)} files) -> {os.path.basename(path)}")
    t0 = time.time()
    if compiler == "nvcc":
        cmd = [nvcc_path()] + NVCC_FLAGS + extra + ["-I", os.path.join(_HERE, "kernels"), "-o", tmp] + srcs
    else:
        cmd = [_find("g++", ["/usr/bin/g++"])] + CXX_FLAGS + extra + ["-I", os.path.join(_HERE, "runtime"),
                                                                 "-o", tmp] + srcs
    try:
        _run(cmd, name)
        os.replace(tmp, path)
    finally:
        if os.path.exists(tmp):
            os.unlink(tmp)
    _say(f"compiled {name} in {time.time() - t0:.1f} s")
    # older binaries of this library are of no use any more
    prefix = f"lib{name}-"
    for f in os.listdir(os.path.dirname(path)):
        if f.startswith(prefix) and f.endswith(".so") and f != os.path.basename(path):
            try:
                os.unlink(os.path.join(os.path.dirname(path), f))
            except OSError:
                pass
    return path


def load(name: str) -> ctypes.CDLL:
    """The library as a ctypes handle, compiled first if needed."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            lib = ctypes.CDLL(build(name))
            _loaded[name] = lib
        return lib


def build_all(force: bool = False) -> list[str]:
    return [build(n, force) for n in LIBRARIES]
