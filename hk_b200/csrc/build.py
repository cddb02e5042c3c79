"""Builds the CUDA sources of this folder for sm_100a with nvcc (and the host-only C++ runtime with the
C++ compiler) and loads them with ctypes.

Every library is one `.cu` file compiled alone (no framework headers, so a file takes
seconds).  Built files live in `_build/` beside the sources, named by a hash of the
source text and flags, so a changed source is rebuilt and a built file is found again
by the next process.  A library is compiled when it is first asked for: a model that
runs in 32-bit never compiles the bfloat16 tensor-core kernels.  While nvcc runs, a
line goes to stderr now and then.  There is no fallback: without nvcc, or when a
source does not compile, `load` raises.
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
from typing import Dict, List

HERE = os.path.dirname(os.path.abspath(__file__))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]

# library name -> source file; headers every library depends on
LIBRARIES: Dict[str, str] = {
    "elementwise": "elementwise.cu",
    "gemm_generic": "gemm_generic.cu",
    "attention_generic": "attention_generic.cu",
    "sampling": "sampling.cu",
    "random_init": "random_init.cu",
    "gemm_tc": "gemm_tc.cu",
    "gemm_smallm": "gemm_smallm.cu",
    "gemm_stream": "gemm_stream.cu",
    "attention_flash": "attention_flash.cu",
    "attention_prefill_tc": "attention_prefill_tc.cu",
    "runtime": "runtime.cpp",          # host only: the cache's books (no GPU code, no CUDA headers)
}


def libraries_for(bfloat16: bool) -> List[str]:
    """The kernel libraries a model needs: the generic ones always (the 32-bit path, and shapes the fast kernels
    refuse), the tensor-core and streaming ones only when it computes in bfloat16."""
    needed = ["elementwise", "gemm_generic", "attention_generic"]
    if bfloat16:
        needed += ["gemm_smallm", "gemm_stream", "gemm_tc", "attention_flash", "attention_prefill_tc"]
    return needed


HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden"]
HEADERS: List[str] = ["common.cuh", "attention_noalloc.h"]

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()
_dir_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    cands = []
    if os.environ.get("HK_B200_NVCC"):
        cands.append(os.environ["HK_B200_NVCC"])
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            cands.append(os.path.join(os.environ[var], "bin", "nvcc"))
    cands.append("/usr/local/cuda/bin/nvcc")
    w = shutil.which("nvcc")
    if w:
        cands.append(w)
    for c in cands:
        if os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise BuildError("nvcc was not found (looked at HK_B200_NVCC, CUDA_HOME, /usr/local/cuda, PATH); "
                     "the CUDA kernels cannot be built and there is no fallback")


def find_cxx() -> str:
    cands = [os.environ.get("HK_B200_CXX"), os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")]
    for c in cands:
        if c and (os.path.isfile(c) or shutil.which(c)):
            return c
    raise BuildError("no C++ compiler was found (looked at HK_B200_CXX, CXX, g++, c++, clang++); the runtime library cannot be built")


def _is_host(name: str) -> bool:
    return LIBRARIES[name].endswith(".cpp")


_build_dir = None


def build_dir() -> str:
    """The folder of the built files: `_build/` beside the sources, or a per-user folder under the temporary
    directory when that cannot be written (a checkout that belongs to someone else).  Decided once per process."""
    global _build_dir
    with _dir_lock:
        if _build_dir is None:
            d = os.environ.get("HK_B200_BUILD_DIR") or os.path.join(HERE, "_build")
            try:
                os.makedirs(d, exist_ok=True)
                probe = os.path.join(d, f".w{os.getpid()}.{threading.get_ident()}")
                with open(probe, "w"):
                    pass
                os.unlink(probe)
            except OSError:
                d = os.path.join(tempfile.gettempdir(), f"hk_b200_build_{os.getuid()}")
                os.makedirs(d, exist_ok=True)
            _build_dir = d
        return _build_dir


def _extra_flags() -> List[str]:
    """Extra nvcc flags from HK_B200_NVCC_FLAGS (for instance -Xptxas -v); they are part of a built file's name."""
    return os.environ.get("HK_B200_NVCC_FLAGS", "").split()


def _digest(name: str) -> str:
    h = hashlib.sha256()
    for fn in [LIBRARIES[name]] + ([] if _is_host(name) else HEADERS):
        with open(os.path.join(HERE, fn), "rb") as f:
            h.update(f.read())
    h.update(" ".join(HOST_FLAGS if _is_host(name) else NVCC_FLAGS + _extra_flags()).encode())
    return h.hexdigest()[:16]


def library_path(name: str) -> str:
    return os.path.join(build_dir(), f"libhk_{name}.{_digest(name)}.so")


def _say(msg: str) -> None:
    print(f"[hk_b200] {msg}", file=sys.stderr, flush=True)


def build(name: str, verbose: bool = True) -> str:
    """Compiles library `name` if its built file is absent; returns the file's path."""
    if name not in LIBRARIES:
        raise BuildError(f"no library named '{name}'")
    out = library_path(name)
    if os.path.isfile(out):
        return out
    src = os.path.join(HERE, LIBRARIES[name])
    tmp = f"{out}.{os.getpid()}.tmp"
    if _is_host(name):
        cmd = [find_cxx()] + HOST_FLAGS + ["-o", tmp, src]
    else:
        cmd = [find_nvcc()] + NVCC_FLAGS + _extra_flags() + ["-I", HERE, "-o", tmp, src]
    if verbose:
        _say(f"compiling {LIBRARIES[name]}" + ("" if _is_host(name) else " for sm_100a") + " ...")
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            if verbose:
                _say(f"still compiling {LIBRARIES[name]} ({time.time() - t0:.0f} s)")

    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    try:
        log, _ = proc.communicate()
    finally:
        done.set()
    if proc.returncode != 0:
        try:
            os.unlink(tmp)
        except OSError:
            pass
        raise BuildError(f"{os.path.basename(cmd[0])} failed on {LIBRARIES[name]} (exit {proc.returncode}):\n{log}")
    os.replace(tmp, out)
    if verbose:
        _say(f"built {os.path.basename(out)} in {time.time() - t0:.1f} s")
    return out


def build_many(names, verbose: bool = True) -> None:
    """Compiles several libraries side by side (one nvcc process each)."""
    errors = []
    threads = []

    def run(n):
        try:
            build(n, verbose)
        except Exception as e:  # noqa: BLE001 - reported below
            errors.append(e)

    for n in names:
        if not os.path.isfile(library_path(n)):
            t = threading.Thread(target=run, args=(n,))
            t.start()
            threads.append(t)
    for t in threads:
        t.join()
    if errors:
        raise errors[0]


def load(name: str) -> ctypes.CDLL:
    """The loaded library `name`, compiled first if need be."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            lib = ctypes.CDLL(build(name))
            _loaded[name] = lib
        return lib
