"""Compiling and loading the sm_100a kernels.

Each `.cu` file of this folder becomes one shared library, built with nvcc for
`sm_100a` and loaded through ctypes.  A library is built the first time one of
its functions is needed (so a run compiles only what its model and precision
use) and kept beside the sources in `_build/`, or under the system's temporary
folder when the source tree cannot be written.  A library is rebuilt when its
source, a header it includes, or the flags change.

There is no fallback: if nvcc is missing or a build fails the error is raised
to the caller, and nothing here computes on the CPU.
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
from typing import Dict, List, Optional

_HERE = os.path.dirname(os.path.abspath(__file__))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]

# Every library and the sources (beside the headers) it is made of.
LIBRARIES: Dict[str, List[str]] = {
    "rowwise": ["rowwise.cu"],
    "gemm_plain": ["gemm_plain.cu"],
    "attention_plain": ["attention_plain.cu"],
    "gemm_tc": ["gemm_tc.cu"],
    "gemm_tc_pair": ["gemm_tc_pair.cu"],
    "attention_decode": ["attention_decode.cu"],
    "attention_prefill": ["attention_prefill.cu"],
    "attention_prefill_tc": ["attention_prefill_tc.cu"],
    "sampling": ["sampling.cu"],
    "selftest": ["selftest.cu"],              # the bounded wait made to run out on purpose (tests)
    "runtime": ["runtime/runtime.cpp", "runtime/engine.cpp", "runtime/loader.cpp"],       # host code: the parts' forward passes (no kernels of its own)
}

_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}


class BuildError(RuntimeError):
    """A kernel library could not be compiled or loaded."""


def _nvcc() -> str:
    for cand in (os.environ.get("LLMX_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc was not found (looked at $LLMX_NVCC, PATH and /usr/local/cuda/bin); "
                     "the kernels cannot be built and there is no other path")


_build_dir_cache: Optional[str] = None
_dir_lock = threading.Lock()


def _build_dir() -> str:
    global _build_dir_cache
    with _dir_lock:
        if _build_dir_cache is None:
            _build_dir_cache = _find_build_dir()
        return _build_dir_cache


def _find_build_dir() -> str:
    for cand in (os.environ.get("LLMX_BUILD_DIR"), os.path.join(_HERE, "_build")):
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
    d = os.path.join(tempfile.gettempdir(), f"llmx_b200_build_{os.getuid()}")
    os.makedirs(d, exist_ok=True)
    return d


def _includes(path: str, seen: set) -> None:
    """The local headers `path` includes, recursively."""
    with open(path, "r", encoding="utf-8") as fh:
        for line in fh:
            line = line.strip()
            if line.startswith("#include \""):
                for base in (os.path.dirname(path), _HERE):
                    inc = os.path.normpath(os.path.join(base, line.split('"')[1]))
                    if os.path.exists(inc):
                        if inc not in seen:
                            seen.add(inc)
                            _includes(inc, seen)
                        break


def _digest(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    files = [os.path.join(_HERE, f) for f in LIBRARIES[name]]
    headers: set = set()
    for f in files:
        _includes(f, headers)
    for f in files + sorted(headers):
        with open(f, "rb") as fh:
            h.update(os.path.basename(f).encode())
            h.update(fh.read())
    return h.hexdigest()[:16]


def library_path(name: str) -> str:
    return os.path.join(_build_dir(), f"llmx_{name}_{_digest(name)}.so")


def _remove_older_builds(name: str, keep: str) -> None:
    """Older builds of library `name` beside `keep` are of no further use.  A build's file is the library's name and 16
    hex digits of digest: `llmx_gemm_tc_pair_<digest>.so` is no older build of `gemm_tc`."""
    older = re.compile(rf"llmx_{re.escape(name)}_[0-9a-f]{{16}}\.so")
    folder = os.path.dirname(keep)
    for f in os.listdir(folder):
        if older.fullmatch(f) and os.path.join(folder, f) != keep:
            try:
                os.remove(os.path.join(folder, f))
            except OSError:
                pass


def build(name: str, verbose: bool = True) -> str:
    """Compile library `name` if its up-to-date build is missing; return the path."""
    if name not in LIBRARIES:
        raise BuildError(f"no kernel library named {name!r}")
    out = library_path(name)
    if os.path.exists(out):
        return out
    nvcc = _nvcc()
    srcs = [os.path.join(_HERE, s) for s in LIBRARIES[name]]
    tmp = f"{out}.{os.getpid()}.tmp"
    cmd = [nvcc] + NVCC_FLAGS + ["-I", _HERE, "-o", tmp] + srcs + (["-ldl"] if name == "runtime" else [])
    if verbose:
        print(f"[llmx_b200] compiling {name} for sm_100a ...", file=sys.stderr, flush=True)
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    # A line now and then while nvcc works, so a first call does not look hung.
    while True:
        try:
            log, _ = proc.communicate(timeout=15)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[llmx_b200] still compiling {name} ({time.time() - t0:.0f} s)", file=sys.stderr, flush=True)
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise BuildError(f"nvcc failed for {name}:\n{' '.join(cmd)}\n{log}")
    os.replace(tmp, out)
    _remove_older_builds(name, out)
    if verbose:
        print(f"[llmx_b200] compiled {name} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return out


def load(name: str) -> ctypes.CDLL:
    """The loaded library `name`, building it first if needed."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = build(name)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise BuildError(f"cannot load {path}: {e}") from None
            _loaded[name] = lib
        return lib


def build_all(verbose: bool = True, jobs: int = 4) -> Dict[str, str]:
    """Compile every library (a few at a time); returns name -> path."""
    from concurrent.futures import ThreadPoolExecutor
    names = [n for n in LIBRARIES if all(os.path.exists(os.path.join(_HERE, s)) for s in LIBRARIES[n])]
    with ThreadPoolExecutor(max_workers=jobs) as pool:
        paths = list(pool.map(lambda n: build(n, verbose), names))
    return dict(zip(names, paths))
