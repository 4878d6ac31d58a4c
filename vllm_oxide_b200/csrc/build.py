"""Builds and loads the engine's native libraries, one shared object per source module.

Each `.cu` file under this folder is a module with a plain C interface (no torch headers,
so a file compiles in seconds); each `.cpp` under `runtime/` builds into one pybind11
module. A library is compiled at its first use for sm_100a, kept beside the sources in
`_build/`, and rebuilt when its sources or flags change. There is no fallback: if a
library cannot be built or loaded, the caller gets a `KernelError`.
"""
from __future__ import annotations

import ctypes
import hashlib
import importlib.util
import os
import shutil
import subprocess
import sys
import sysconfig
import tempfile
import threading
import time
from typing import Dict, List

from ..errors import KernelError

_HERE = os.path.dirname(os.path.abspath(__file__))
# No fast-math flag: division, sqrt, exp, sin and cos keep nvcc's precise defaults.
_NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
               "-Xcompiler", "-fPIC", "-shared", "-Xptxas", "-v"]
if os.environ.get("VOB_TIMELINE") == "1":      # per-kernel timeline recording (see common.cuh); a different build
    _NVCC_FLAGS = _NVCC_FLAGS + ["-DVOB_TIMELINE"]
_CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall"]

CUDA_MODULES = ("elementwise", "gemm_f32", "attention", "attention_mma", "attention_sm100", "sampling", "gemm_sm100", "gemm_sm100_pair")
_lock = threading.Lock()
_loaded: Dict[str, object] = {}


_bdir = None
_bdir_lock = threading.Lock()


def _build_dir() -> str:
    """`_build/` beside the sources; a per-user folder under the temp dir if that is read-only."""
    global _bdir
    with _bdir_lock:
        if _bdir is None:
            d = os.path.join(_HERE, "_build")
            try:
                os.makedirs(d, exist_ok=True)
                fd, probe = tempfile.mkstemp(dir=d)
                os.close(fd)
                os.remove(probe)
            except OSError:
                d = os.path.join(tempfile.gettempdir(), f"vllm_oxide_b200-build-{os.getuid()}")
                os.makedirs(d, exist_ok=True)
            _bdir = d
        return _bdir


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise KernelError("nvcc was not found (set NVCC or put it on PATH); the CUDA kernels cannot be built")


def _digest(paths: List[str], flags: List[str]) -> str:
    h = hashlib.sha256()
    for p in paths:
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:20]


def _run(cmd: List[str], what: str) -> str:
    """Run a compiler, printing a line every few seconds so a first call does not look hung."""
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    out: List[str] = []
    reader = threading.Thread(target=lambda: out.extend(proc.stdout.readlines()), daemon=True)
    reader.start()
    while proc.poll() is None:
        try:
            proc.wait(timeout=10)
        except subprocess.TimeoutExpired:
            print(f"[vllm_oxide_b200] still compiling {what} ({int(time.time() - t0)} s)", file=sys.stderr, flush=True)
    reader.join()
    text = "".join(out)
    if proc.returncode != 0:
        raise KernelError(f"building {what} failed (exit {proc.returncode}):\n{' '.join(cmd)}\n{text[-4000:]}")
    return text


def _headers() -> List[str]:
    return sorted(os.path.join(_HERE, f) for f in os.listdir(_HERE) if f.endswith((".cuh", ".h")))


def cuda_library_path(module: str, build: bool = True) -> str:
    """Path of the shared object of one `.cu` module, compiling it if stale."""
    src = os.path.join(_HERE, module + ".cu")
    if not os.path.exists(src):
        raise KernelError(f"no kernel source {src}")
    deps = [src] + _headers()
    tag = _digest(deps, _NVCC_FLAGS)
    bdir = _build_dir()
    so = os.path.join(bdir, f"libvob200_{module}.{tag}.so")
    if os.path.exists(so) or not build:
        return so
    for old in os.listdir(bdir):
        if old.startswith(f"libvob200_{module}.") and old.endswith((".so", ".log")):
            try:
                os.remove(os.path.join(bdir, old))
            except OSError:
                pass
    print(f"[vllm_oxide_b200] compiling CUDA module '{module}' for sm_100a ...", file=sys.stderr, flush=True)
    tmp = so + f".{os.getpid()}.tmp"
    log = _run([_nvcc()] + _NVCC_FLAGS + ["-I", _HERE, "-o", tmp, src], f"{module}.cu")
    with open(os.path.join(bdir, f"libvob200_{module}.{tag}.log"), "w") as f:
        f.write(log)
    os.replace(tmp, so)
    print(f"[vllm_oxide_b200] built {os.path.basename(so)}", file=sys.stderr, flush=True)
    return so


def load_cuda_module(module: str) -> ctypes.CDLL:
    """dlopen one kernel module (building it first if needed)."""
    with _lock:
        if module not in _loaded:
            path = cuda_library_path(module)
            try:
                _loaded[module] = ctypes.CDLL(path)
            except OSError as e:
                raise KernelError(f"cannot load kernel library {path}: {e}") from e
        return _loaded[module]


def runtime_module():
    """Import the native host runtime (cache manager, scheduler, batch builder), building the
    pybind11 module first if needed."""
    with _lock:
        if "runtime" in _loaded:
            return _loaded["runtime"]
        import pybind11
        rdir = os.path.join(_HERE, "runtime")
        srcs = sorted(os.path.join(rdir, f) for f in os.listdir(rdir) if f.endswith(".cpp"))
        hdrs = sorted(os.path.join(rdir, f) for f in os.listdir(rdir) if f.endswith((".h", ".hpp")))
        tag = _digest(srcs + hdrs, _CXX_FLAGS + [sys.version])
        bdir = _build_dir()
        so = os.path.join(bdir, f"vob200_runtime_{tag}.so")
        if not os.path.exists(so):
            for old in os.listdir(bdir):
                if old.startswith("vob200_runtime_") and old.endswith(".so"):
                    try:
                        os.remove(os.path.join(bdir, old))
                    except OSError:
                        pass
            cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
            if not cxx:
                raise KernelError("no C++ compiler found (g++); the host runtime cannot be built")
            print("[vllm_oxide_b200] compiling the host runtime (C++) ...", file=sys.stderr, flush=True)
            tmp = so + f".{os.getpid()}.tmp"
            _run([cxx] + _CXX_FLAGS + [f"-DVOB_MODULE_NAME=vob200_runtime_{tag}",
                  "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], "-I", rdir,
                  "-o", tmp] + srcs, "runtime")
            os.replace(tmp, so)
        spec = importlib.util.spec_from_file_location(f"vob200_runtime_{tag}", so)
        try:
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
        except ImportError as e:
            raise KernelError(f"cannot load the host runtime {so}: {e}") from e
        _loaded["runtime"] = mod
        return mod


def ensure_built(modules) -> None:
    """Compile the given CUDA modules (those that are stale) side by side, so that a first call
    waits for the slowest file rather than for the sum."""
    errors: List[str] = []

    def one(m):
        try:
            cuda_library_path(m)
        except KernelError as e:
            errors.append(str(e))

    threads = [threading.Thread(target=one, args=(m,)) for m in modules]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise KernelError("\n\n".join(errors))


def build_all(verbose: bool = True) -> None:
    """Compile every module (in parallel); used by the build check and before a GPU run."""
    errors: List[str] = []

    def one(m):
        try:
            cuda_library_path(m)
        except KernelError as e:
            errors.append(str(e))

    mods = [m for m in CUDA_MODULES if os.path.exists(os.path.join(_HERE, m + ".cu"))]
    threads = [threading.Thread(target=one, args=(m,)) for m in mods]
    for t in threads:
        t.start()
    try:
        runtime_module()
    except KernelError as e:
        errors.append(str(e))
    for t in threads:
        t.join()
    if errors:
        raise KernelError("\n\n".join(errors))


def ptxas_log(module: str) -> str:
    """The compiler's register / spill / shared-memory report of a built module."""
    so = cuda_library_path(module)
    with open(so[:-3] + ".log") as f:
        return f.read()
