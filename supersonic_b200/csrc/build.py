"""Compiles the ``.cu`` files beside this module with nvcc for sm_100a, one shared
library each, and loads them with ctypes; the host runtime (``../host/runtime.cpp``, plain
C++ without CUDA) is built the same way with the C++ compiler.

A library is built the first time something asks for it (so a run compiles only
what its model needs) and again whenever its sources or flags change; a progress
line goes to stderr every few seconds meanwhile.  Libraries live in ``_build/``
beside the sources, or in a per-user temporary folder when that is not
writable.  The reference compiles its bridges from ``build.rs`` with
``-std=c++17 -O3 --use_fast_math`` for one detected architecture
(crates/kernel-ffi/build.rs:284-363); here the only target is sm_100a and
fast-math is a per-file choice (never for the float32 kernels).
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
from typing import Dict, List

_HERE = os.path.dirname(os.path.abspath(__file__))

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC", "-shared",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fvisibility=hidden"]

# library name -> (source files, extra nvcc flags, extra link flags)
LIBRARIES: Dict[str, Dict[str, List[str]]] = {
    "plain_ops": {"sources": ["plain_ops.cu"], "flags": [], "link": []},
    "sampling": {"sources": ["sampling.cu"], "flags": [], "link": []},
    "decode_ops": {"sources": ["decode_ops.cu"], "flags": [], "link": []},
    "prefill_attention": {"sources": ["prefill_attention.cu"], "flags": [], "link": []},
    "prefill_attention_tc": {"sources": ["prefill_attention_tc.cu"], "flags": [], "link": []},
    "elementwise_ops": {"sources": ["elementwise_ops.cu"], "flags": [], "link": []},
    "gemv_tc": {"sources": ["gemv_tc.cu"], "flags": [], "link": []},
    "gemm_tc": {"sources": ["gemm_tc.cu"], "flags": [], "link": []},
    "attention_decode_static": {"sources": ["attention_decode_static.cu"], "flags": [], "link": []},
    "random_fill": {"sources": ["random_fill.cu"], "flags": [], "link": []},
    # the host side's native core: no CUDA in it, so it is compiled by the C++ compiler alone
    "host_runtime": {"sources": ["runtime.cpp"], "flags": [], "link": [], "dir": os.path.join(os.path.dirname(_HERE), "host"),
                     "compiler": "c++"},
}
HOST_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall"]
_INCLUDE = re.compile(r'^\s*#\s*include\s+"([^"]+)"', re.M)


def _sources_of(name: str) -> List[str]:
    """The library's sources and every header beside them that they include, directly or not: what its
    digest is taken over, so that a change to one kernel's header rebuilds only the libraries that use it."""
    todo, seen = list(LIBRARIES[name]["sources"]), []
    base = _dir_of(name)
    while todo:
        f = todo.pop()
        if f in seen:
            continue
        seen.append(f)
        with open(os.path.join(base, f), "r", encoding="utf-8") as fh:
            for inc in _INCLUDE.findall(fh.read()):
                if os.path.isfile(os.path.join(base, inc)):
                    todo.append(inc)
    return sorted(seen)


def _dir_of(name: str) -> str:
    return LIBRARIES[name].get("dir", _HERE)


def _flags_of(name: str) -> List[str]:
    spec = LIBRARIES[name]
    base = HOST_FLAGS if spec.get("compiler") == "c++" else ARCH_FLAGS + BASE_FLAGS
    return base + spec["flags"] + spec["link"]

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def register_library(name: str, sources: List[str], flags: List[str] = (), link: List[str] = ()):
    LIBRARIES[name] = {"sources": list(sources), "flags": list(flags), "link": list(link)}


def find_cxx() -> str:
    for cand in (os.environ.get("SSB200_CXX"), os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"),
                 shutil.which("clang++")):
        if cand and (os.path.isfile(cand) or shutil.which(cand)):
            return cand
    raise BuildError("no C++ compiler found (looked at $SSB200_CXX, $CXX, g++, c++, clang++): "
                     "the host runtime cannot be built and there is no other path")


def find_nvcc() -> str:
    for cand in (os.environ.get("SSB200_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $SSB200_NVCC, $CUDA_HOME/bin, PATH, /usr/local/cuda/bin); "
                     "the CUDA kernels cannot be built and there is no other path")


def _build_dir() -> str:
    env = os.environ.get("SSB200_BUILD_DIR")
    cands = [env] if env else []
    cands.append(os.path.join(_HERE, "_build"))
    cands.append(os.path.join(tempfile.gettempdir(), f"supersonic_b200-build-{os.getuid()}"))
    for d in cands:
        try:
            os.makedirs(d, exist_ok=True)
            fd, probe = tempfile.mkstemp(prefix=".w", dir=d)
            os.close(fd)
            os.remove(probe)
            return d
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {cands}")


def _digest(name: str) -> str:
    spec = LIBRARIES[name]
    h = hashlib.sha256()
    for f in _sources_of(name):
        with open(os.path.join(_dir_of(name), f), "rb") as fh:
            h.update(f.encode() + b"\0" + fh.read())
    h.update(" ".join(_flags_of(name)).encode())
    return h.hexdigest()[:20]


def library_path(name: str) -> str:
    """Where the library is, or would be built; looks in every candidate folder for a
    library whose recorded digest matches the sources."""
    digest = _digest(name)
    fname = f"libssb200_{name}.so"
    for d in (os.environ.get("SSB200_BUILD_DIR"), os.path.join(_HERE, "_build"),
              os.path.join(tempfile.gettempdir(), f"supersonic_b200-build-{os.getuid()}")):
        if not d:
            continue
        so, stamp = os.path.join(d, fname), os.path.join(d, fname + ".digest")
        try:
            if os.path.isfile(so) and open(stamp).read().strip() == digest:
                return so
        except OSError:
            pass
    return ""


def build_library(name: str, verbose: bool = True, force: bool = False) -> str:
    """Compile ``name`` if it is missing or stale; returns the path of the library."""
    if name not in LIBRARIES:
        raise BuildError(f"unknown kernel library {name!r}; known: {sorted(LIBRARIES)}")
    if not force:
        so = library_path(name)
        if so:
            return so
    spec = LIBRARIES[name]
    out_dir = _build_dir()
    so = os.path.join(out_dir, f"libssb200_{name}.so")
    tmp = so + f".{os.getpid()}.tmp"
    src_dir = _dir_of(name)
    if spec.get("compiler") == "c++":
        cmd = ([find_cxx()] + HOST_FLAGS + spec["flags"] + ["-I", src_dir]
               + [os.path.join(src_dir, s) for s in spec["sources"]] + spec["link"] + ["-o", tmp])
    else:
        cmd = ([find_nvcc()] + ARCH_FLAGS + BASE_FLAGS + spec["flags"] + ["-I", src_dir]
               + [os.path.join(src_dir, s) for s in spec["sources"]] + spec["link"] + ["-o", tmp])
    if verbose:
        print(f"[supersonic_b200] compiling {name}" + ("" if spec.get("compiler") == "c++" else " for sm_100a") + " ...",
              file=sys.stderr, flush=True)
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                            cwd=out_dir)
    done = threading.Event()

    def _tick():
        while not done.wait(10.0):
            if verbose:
                print(f"[supersonic_b200] still compiling {name} ({time.time() - t0:.0f} s)",
                      file=sys.stderr, flush=True)
    ticker = threading.Thread(target=_tick, daemon=True)
    ticker.start()
    try:
        out, _ = proc.communicate()
    finally:
        done.set()
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise BuildError(f"the compiler failed for {name} (exit {proc.returncode}):\n{' '.join(cmd)}\n{out}")
    os.replace(tmp, so)
    with open(so + ".digest", "w") as f:
        f.write(_digest(name) + "\n")
    if verbose:
        print(f"[supersonic_b200] built {name} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return so


def build_all(verbose: bool = True, force: bool = False) -> List[str]:
    """Compile every registered library (several at once)."""
    names = sorted(LIBRARIES)
    results: Dict[str, object] = {}

    def _one(n):
        try:
            results[n] = build_library(n, verbose, force)
        except Exception as e:       # noqa: BLE001 - reported below
            results[n] = e
    threads = [threading.Thread(target=_one, args=(n,)) for n in names]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    errors = [f"{n}: {r}" for n, r in results.items() if isinstance(r, Exception)]
    if errors:
        raise BuildError("\n".join(errors))
    return [results[n] for n in names]


def load_library(name: str) -> ctypes.CDLL:
    """The loaded library, built first if needed.  Fails loudly: there is no fallback."""
    with _lock:
        if name not in _loaded:
            so = build_library(name)
            try:
                _loaded[name] = ctypes.CDLL(so, mode=ctypes.RTLD_LOCAL)
            except OSError as e:
                raise BuildError(f"cannot load {so}: {e}") from None
        return _loaded[name]
