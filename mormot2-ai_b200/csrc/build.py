"""Compiles the CUDA sources of this folder for sm_100a with nvcc and loads them.

Each ``.cu`` file becomes one shared library with a C interface, built in place under
``csrc/_build/`` (or, if that folder cannot be written, under a per-user folder in the
system's temporary folder) and loaded with ``ctypes``. A library is compiled when it is first
asked for, so a model compiles what it needs; a line is printed now and then meanwhile.
There is no fallback: a missing compiler or a failed build raises ``KernelError``.
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

from ..errors import KernelError

HERE = os.path.dirname(os.path.abspath(__file__))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]

# more flags for nvcc, e.g. MORMOT_B200_NVCC_FLAGS="-DMB_WAIT_LIMIT=1024" (the iteration limit of
# the kernels' bounded waits); they are part of the built library's name
NVCC_FLAGS += os.environ.get("MORMOT_B200_NVCC_FLAGS", "").split()
# MORMOT_B200_DEBUG=1: the build whose kernels check every index into a page table before they
# use it (csrc/common.cuh); Runtime.check then also asks every library for what it found
DEBUG_BOUNDS = os.environ.get("MORMOT_B200_DEBUG", "") not in ("", "0")
if DEBUG_BOUNDS:
    NVCC_FLAGS.append("-DMB_DEBUG_BOUNDS")

# library name -> source file; headers that every library depends on
SOURCES = {
    "elementwise": "elementwise.cu",
    "rope": "rope.cu",
    "gemm_simt": "gemm_simt.cu",
    "attention_simt": "attention_simt.cu",
    "sampling": "sampling.cu",
    "gemm_tc": "gemm_tc.cu",
    "attention_mma": "attention_mma.cu",
    "attention_tc": "attention_tc.cu",
}
HEADERS = ["common.cuh"]
EXTRA_HEADERS = {"gemm_tc": ["tc_common.cuh"],
                 "attention_mma": ["mma_common.cuh", "tc_common.cuh", "no_alloc.h"],
                 "attention_tc": ["tc_common.cuh"]}

_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise KernelError("nvcc was not found (PATH, $NVCC, /usr/local/cuda/bin): the kernels "
                      "of this library cannot be built, and there is no other code path")


_build_dir: Optional[str] = None


def build_dir() -> str:
    global _build_dir
    with _lock:
        if _build_dir is None:
            _build_dir = _find_build_dir()
        return _build_dir


def _find_build_dir() -> str:
    override = os.environ.get("MORMOT_B200_BUILD_DIR")
    cands = [override] if override else []
    cands.append(os.path.join(HERE, "_build"))
    cands.append(os.path.join(tempfile.gettempdir(), f"mormot2-ai_b200-build-{os.getuid()}"))
    for d in cands:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".probe-{os.getpid()}")
            with open(probe, "w"):
                pass
            os.unlink(probe)
            return d
        except OSError:
            continue
    raise KernelError(f"no folder to build the kernels in (tried {', '.join(cands)})")


def _digest(name: str) -> str:
    """Names a build: the sources' digest, then the flags' digest."""
    h = hashlib.sha256()
    for fn in [SOURCES[name]] + HEADERS + EXTRA_HEADERS.get(name, []):
        path = os.path.join(HERE, fn)
        if os.path.isfile(path):
            with open(path, "rb") as f:
                h.update(f.read())
    return h.hexdigest()[:16] + "-" + _flags_digest()


def _flags_digest() -> str:
    return hashlib.sha256(" ".join(NVCC_FLAGS).encode()).hexdigest()[:6]


def library_path(name: str) -> str:
    return os.path.join(build_dir(), f"libmb_{name}-{_digest(name)}.so")


def compile_library(name: str, verbose: bool = True) -> str:
    """Builds one library if it is not there yet; returns its path."""
    if name not in SOURCES:
        raise KernelError(f"no kernel library \"{name}\"")
    out = library_path(name)
    if os.path.isfile(out):
        return out
    src = os.path.join(HERE, SOURCES[name])
    if not os.path.isfile(src):
        raise KernelError(f"the source {src} is missing")
    tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [nvcc_path()] + NVCC_FLAGS + ["-o", tmp, src]
    t0 = time.time()
    if verbose:
        print(f"[mormot2-ai_b200] compiling {SOURCES[name]} for sm_100a ...", file=sys.stderr,
              flush=True)
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, cwd=HERE)
    last = t0
    while True:
        try:
            log, _ = proc.communicate(timeout=5)
            break
        except subprocess.TimeoutExpired:
            if verbose and time.time() - last >= 10:
                last = time.time()
                print(f"[mormot2-ai_b200] ... still compiling {SOURCES[name]} "
                      f"({int(last - t0)} s)", file=sys.stderr, flush=True)
    if proc.returncode != 0:
        try:
            os.unlink(tmp)
        except OSError:
            pass
        raise KernelError(f"nvcc failed on {SOURCES[name]}:\n{log.decode(errors='replace')}")
    os.replace(tmp, out)
    # builds of older sources of this library with the same flags are of no use any more (a
    # build with other flags, the debug build for one, stays beside this one)
    prefix, suffix = f"libmb_{name}-", f"-{_flags_digest()}.so"
    for fn in os.listdir(os.path.dirname(out)):
        if fn.startswith(prefix) and fn.endswith(suffix) and fn != os.path.basename(out):
            try:
                os.unlink(os.path.join(os.path.dirname(out), fn))
            except OSError:
                pass
    if verbose:
        print(f"[mormot2-ai_b200] compiled {SOURCES[name]} in {time.time() - t0:.1f} s",
              file=sys.stderr, flush=True)
    return out


def compile_libraries(names: Iterable[str], verbose: bool = True) -> List[str]:
    """Builds several libraries side by side."""
    names = list(names)
    results: Dict[str, object] = {}

    def work(n):
        try:
            results[n] = compile_library(n, verbose)
        except Exception as e:  # noqa: BLE001 - re-raised below
            results[n] = e

    threads = [threading.Thread(target=work, args=(n,)) for n in names]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for n in names:
        if isinstance(results[n], Exception):
            raise results[n]
    return [results[n] for n in names]


def load_library(name: str) -> ctypes.CDLL:
    """The loaded library, compiled first if need be."""
    with _lock:
        if name in _loaded:
            return _loaded[name]
    path = compile_library(name)
    with _lock:
        if name not in _loaded:
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelError(f"cannot load {path}: {e}") from None
            lib.mb_last_error.restype = ctypes.c_char_p
            _loaded[name] = lib
        return _loaded[name]


def debug_faults() -> List[str]:
    """What the loaded libraries of a debug build found since the last call (and forgets it):
    one line per library whose kernels met an index outside its table."""
    if not DEBUG_BOUNDS:
        return []
    with _lock:
        libs = dict(_loaded)
    out = []
    names = {1: "a position outside the slot's row of the page table", 2: "a negative page"}
    for name, lib in libs.items():
        four = (ctypes.c_int * 4)()
        rc = lib.mb_debug_fault(four)
        if rc == 1 and four[0]:
            out.append(f"{name}: {names.get(four[0], 'code %d' % four[0])} "
                       f"({four[1]}, {four[2]}, {four[3]})")
    return out


def build_all(verbose: bool = True) -> List[str]:
    return compile_libraries([n for n in SOURCES
                              if os.path.isfile(os.path.join(HERE, SOURCES[n]))], verbose)
