"""Compiles the CUDA sources of this folder for sm_100a and loads them with ctypes.

Each ``<name>.cu`` becomes ``lib<name>.so`` with a plain C ABI (no torch headers, so a
file compiles in seconds).  A library is built when it is first asked for and its source,
the shared header or the flags have changed since the last build; a line is printed while
that happens.  Libraries are written next to the sources when that folder is writable, else
under a per-user folder in the system's temporary directory.
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
from typing import Dict, Iterable, List, Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "--expt-relaxed-constexpr"]
SOURCES = ("elementwise", "gemm_simt", "attention", "sampling", "gemm_tc", "attention_tc", "attention_fa", "no_alloc")
_EXTRA_LIBS = {}

_lock = threading.Lock()
_dir_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (os.environ.get("EMBER_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (set CUDA_HOME or EMBER_NVCC); the CUDA kernels cannot be built")


def _writable(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe-{os.getpid()}")
        with open(probe, "w") as f:
            f.write("")
        os.remove(probe)
        return True
    except OSError:
        return False


_build_dir_cache: Optional[str] = None


def build_dir() -> str:
    global _build_dir_cache
    with _dir_lock:
        return _build_dir_locked()


def _build_dir_locked() -> str:
    global _build_dir_cache
    if _build_dir_cache:
        return _build_dir_cache
    cands = [os.environ.get("EMBER_BUILD_DIR"), os.path.join(_HERE, "_build"),
             os.path.join(tempfile.gettempdir(), f"ember_b200-build-{os.getuid()}")]
    for c in cands:
        if c and _writable(c):
            _build_dir_cache = c
            return c
    raise BuildError("no writable folder for the compiled kernels (tried: %s)" % ", ".join(x for x in cands if x))


def _digest(name: str) -> str:
    h = hashlib.sha256()
    headers = sorted(f for f in os.listdir(_HERE) if f.endswith((".cuh", ".h")))
    for fn in [name + ".cu"] + headers:
        with open(os.path.join(_HERE, fn), "rb") as f:
            h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + _EXTRA_LIBS.get(name, [])).encode())
    return h.hexdigest()[:16]


def lib_path(name: str) -> str:
    return os.path.join(build_dir(), f"lib{name}.so")


def is_current(name: str) -> bool:
    so, stamp = lib_path(name), lib_path(name) + ".stamp"
    if not (os.path.isfile(so) and os.path.isfile(stamp)):
        return False
    with open(stamp) as f:
        return f.read().strip() == _digest(name)


def compile_one(name: str, verbose: bool = True, ptxas_info: bool = False) -> str:
    """Compiles ``<name>.cu`` if needed; returns the library's path."""
    src = os.path.join(_HERE, name + ".cu")
    if not os.path.isfile(src):
        raise BuildError(f"no such kernel source: {src}")
    so = lib_path(name)
    if is_current(name) and not ptxas_info:
        return so
    nvcc = find_nvcc()
    tmp = f"{so}.{os.getpid()}.tmp"
    cmd = [nvcc] + ARCH_FLAGS + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + \
          ["-I", _HERE, "-o", tmp, src] + _EXTRA_LIBS.get(name, [])
    if verbose:
        print(f"[ember_b200] compiling {name}.cu for sm_100a ...", file=sys.stderr, flush=True)
    t0 = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    out_lines: List[str] = []
    # nvcc prints nothing while it works; report now and then so a first call is not silent
    done = threading.Event()

    def ticker():
        while not done.wait(15.0):
            if verbose:
                print(f"[ember_b200] ... still compiling {name}.cu ({time.time() - t0:.0f} s)", file=sys.stderr, flush=True)

    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    try:
        out, _ = proc.communicate()
    finally:
        done.set()
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise BuildError(f"nvcc failed on {name}.cu:\n{out}")
    os.replace(tmp, so)
    with open(so + ".stamp", "w") as f:
        f.write(_digest(name))
    if verbose:
        print(f"[ember_b200] built lib{name}.so in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    if ptxas_info:
        print(out)
    return so


def build_all(names: Iterable[str] = None, verbose: bool = True) -> List[str]:
    """Compiles every kernel library (in parallel); used by the build check."""
    names = [n for n in (names or SOURCES) if os.path.isfile(os.path.join(_HERE, n + ".cu"))]
    errors: List[str] = []
    paths: Dict[str, str] = {}

    def work(n):
        try:
            paths[n] = compile_one(n, verbose=verbose)
        except BuildError as e:
            errors.append(str(e))

    threads = [threading.Thread(target=work, args=(n,)) for n in names]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise BuildError("\n".join(errors))
    return [paths[n] for n in names]


def load(name: str) -> ctypes.CDLL:
    """The compiled library ``name`` (built first if needed)."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = compile_one(name)
            lib = ctypes.CDLL(path, mode=ctypes.RTLD_LOCAL)
            lib.ember_last_error.restype = ctypes.c_char_p
            _loaded[name] = lib
        return lib
