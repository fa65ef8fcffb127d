"""Compiles the native code in-tree, on first use.

Two kinds of libraries: CUDA kernel libraries built with nvcc for sm_100a and
loaded through ctypes (plain C entry points), and the host runtime built with
g++ as a CPython extension. A library is rebuilt when its sources or flags
change: the file name carries a hash of both. While a compiler runs, a line is
printed every few seconds so that a first call does not look hung.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import importlib.machinery
import importlib.util
import os
import shutil
import subprocess
import sys
import sysconfig
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List

HERE = os.path.dirname(os.path.abspath(__file__))

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall"]

#: kernel libraries: name -> sources under csrc/kernels
KERNEL_LIBS: Dict[str, List[str]] = {
    "garuda_core": ["elementwise.cu", "gemm_simple.cu", "attention_simple.cu", "sampling.cu"],
    "garuda_tc": ["gemm_tcgen05.cu"],
}
HOST_SOURCES = ["cache_manager.cpp", "scheduler.cpp", "step_batch.cpp", "bindings.cpp"]


class BuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[garuda_b200 build] {msg}", file=sys.stderr, flush=True)


def build_dir() -> str:
    """In-tree ``csrc/_build``; a per-user temporary folder if that cannot be written."""
    for cand in (os.environ.get("GARUDA_B200_BUILD_DIR"), os.path.join(HERE, "_build")):
        if not cand:
            continue
        try:
            os.makedirs(cand, exist_ok=True)
            probe = os.path.join(cand, f".w{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return cand
        except OSError:
            continue
    d = os.path.join(tempfile.gettempdir(), f"garuda_b200_build_{os.getuid()}")
    os.makedirs(d, exist_ok=True)
    return d


def _hash(paths: List[str], flags: List[str]) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:12]


def _headers(folder: str) -> List[str]:
    return [os.path.join(folder, f) for f in sorted(os.listdir(folder))
            if f.endswith((".cuh", ".hpp", ".h"))]


def _run(cmd: List[str], what: str) -> None:
    """Run a compiler; print a line every 10 s while it works."""
    done = threading.Event()
    start = time.time()

    def ticker():
        while not done.wait(10.0):
            _log(f"still compiling {what} ({time.time() - start:.0f} s)")

    t = threading.Thread(target=ticker, daemon=True)
    t.start()
    try:
        proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    finally:
        done.set()
    if proc.returncode != 0:
        raise BuildError(f"compiling {what} failed:\n$ {' '.join(cmd)}\n{proc.stdout}")


class _Lock:
    def __init__(self, path):
        self.path = path

    def __enter__(self):
        self.fh = open(self.path, "w")
        fcntl.flock(self.fh, fcntl.LOCK_EX)

    def __exit__(self, *a):
        fcntl.flock(self.fh, fcntl.LOCK_UN)
        self.fh.close()


def _drop_older(out_dir: str, prefix: str, keep: str) -> None:
    """Builds of other versions of the same library (same name, another hash) are deleted, so that
    the folder does not grow with every change of a source. A process that still has one mapped
    keeps it until it exits."""
    for f in os.listdir(out_dir):
        if f.startswith(prefix) and f.endswith(".so") and os.path.join(out_dir, f) != keep:
            try:
                os.remove(os.path.join(out_dir, f))
            except OSError:
                pass


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin): "
                     "the CUDA kernels cannot be built")


def attention_lib_name(head_dim: int) -> str:
    """The tensor-core attention is compiled per head size, when a model first needs it."""
    return f"garuda_attn_hd{int(head_dim)}"


def _lib_recipe(name: str):
    if name.startswith("garuda_attn_hd"):
        return ["attention_mma.cu", "attention_tcgen05.cu", "attention_decode_tma.cu"], [f"-DGB_HEAD_DIM={int(name[len('garuda_attn_hd'):])}"]
    return KERNEL_LIBS[name], []


def kernel_lib_path(name: str) -> str:
    """Build (if needed) and return the path of a kernel library."""
    folder = os.path.join(HERE, "kernels")
    names, defines = _lib_recipe(name)
    sources = [os.path.join(folder, s) for s in names]
    tag = _hash(sources + _headers(folder), NVCC_FLAGS + defines)
    out_dir = build_dir()
    target = os.path.join(out_dir, f"lib{name}.{tag}.so")
    if os.path.exists(target):
        return target
    with _Lock(os.path.join(out_dir, f".{name}.lock")):
        if os.path.exists(target):
            return target
        nvcc = nvcc_path()
        _log(f"compiling {name} for sm_100a ({len(sources)} files; first use only)")
        t0 = time.time()
        objs = []

        def one(src):
            obj = os.path.join(out_dir, f"{name}.{os.path.basename(src)}.{tag}.{os.getpid()}.o")
            _run([nvcc, *NVCC_FLAGS, *defines, "-I", folder, "-c", src, "-o", obj], os.path.basename(src))
            return obj

        with ThreadPoolExecutor(max_workers=min(4, len(sources))) as pool:
            objs = list(pool.map(one, sources))
        tmp = target + f".{os.getpid()}.tmp"
        _run([nvcc, "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a"],
             f"lib{name}")
        os.replace(tmp, target)
        for o in objs:
            try:
                os.remove(o)
            except OSError:
                pass
        _drop_older(out_dir, f"lib{name}.", target)
        _log(f"{name} ready in {time.time() - t0:.0f} s")
    return target


_LOADED: Dict[str, ctypes.CDLL] = {}


def load_kernel_lib(name: str) -> ctypes.CDLL:
    if name not in _LOADED:
        _LOADED[name] = ctypes.CDLL(kernel_lib_path(name))
    return _LOADED[name]


def host_module_path() -> str:
    import pybind11
    folder = os.path.join(HERE, "host")
    sources = [os.path.join(folder, s) for s in HOST_SOURCES]
    includes = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], "-I", folder]
    tag = _hash(sources + _headers(folder), CXX_FLAGS + [sys.version.split()[0], "system-g++"])
    out_dir = build_dir()
    target = os.path.join(out_dir, f"_garuda_host.{tag}.so")
    if os.path.exists(target):
        return target
    with _Lock(os.path.join(out_dir, ".host.lock")):
        if os.path.exists(target):
            return target
        # The system g++: it links libstdc++ dynamically, which an extension that throws
        # exceptions inside a Python process (next to numpy and torch) needs.
        cxx = os.environ.get("GARUDA_B200_CXX") or shutil.which("g++") or "g++"
        _log("compiling the host runtime (first use only)")
        t0 = time.time()

        def one(src):
            obj = os.path.join(out_dir, f"host.{os.path.basename(src)}.{tag}.{os.getpid()}.o")
            _run([cxx, *CXX_FLAGS, *includes, "-c", src, "-o", obj], os.path.basename(src))
            return obj

        with ThreadPoolExecutor(max_workers=len(sources)) as pool:
            objs = list(pool.map(one, sources))
        tmp = target + f".{os.getpid()}.tmp"
        _run([cxx, "-shared", "-o", tmp, *objs], "_garuda_host")
        os.replace(tmp, target)
        for o in objs:
            try:
                os.remove(o)
            except OSError:
                pass
        _drop_older(out_dir, "_garuda_host.", target)
        _log(f"host runtime ready in {time.time() - t0:.0f} s")
    return target


_HOST = None


def load_host_module():
    global _HOST
    if _HOST is None:
        path = host_module_path()
        loader = importlib.machinery.ExtensionFileLoader("_garuda_host", path)
        spec = importlib.util.spec_from_file_location("_garuda_host", path, loader=loader)
        mod = importlib.util.module_from_spec(spec)
        loader.exec_module(mod)
        _HOST = mod
    return _HOST


def build_all(head_dims=(16, 32, 48, 64, 128)) -> None:
    """Everything, for a build check."""
    host_module_path()
    for name in KERNEL_LIBS:
        kernel_lib_path(name)
    for hd in head_dims:
        kernel_lib_path(attention_lib_name(hd))
