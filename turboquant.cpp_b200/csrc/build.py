"""Compiles the kernel files for sm_100a with nvcc and loads them through ctypes.

Each ``.cu`` file becomes one shared library with plain C entry points.  A
library is built the first time something needs it, so a program compiles what
its model uses and nothing else; a line on stderr says what is being compiled
and another one when it is done.  Libraries are kept in ``csrc/_build`` inside
the package when that folder can be written, otherwise in a per-user folder
under the system's temporary directory; the file name carries a hash of the
sources and flags, so a stale library is never loaded.

There is no fallback: if nvcc is missing, a file does not compile or a library
does not load, the caller gets a ``KernelBuildError``.
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

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

# extra flags per kernel file (libraries to link, include paths)
EXTRA_FLAGS: Dict[str, List[str]] = {}

# TQ_DEBUG_INDEX=1 in the environment builds and loads the kernels with their index checks compiled in
# (common.cuh: TQ_CHECKED); the libraries of the two builds carry different hashes and live side by side.
DEBUG_INDEX = os.environ.get("TQ_DEBUG_INDEX", "") not in ("", "0")


def _flags(name: str, debug_index: Optional[bool] = None) -> List[str]:
    debug = DEBUG_INDEX if debug_index is None else debug_index
    return NVCC_FLAGS + (["-DTQ_DEBUG_INDEX"] if debug else []) + EXTRA_FLAGS.get(name, [])

_HEADERS = ["common.cuh"]


class KernelBuildError(RuntimeError):
    pass


_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}


def _say(msg: str) -> None:
    print(f"[turboquant.cpp_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("TQ_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError("nvcc not found (looked at $TQ_NVCC, PATH and /usr/local/cuda/bin); "
                           "the CUDA kernels cannot be built and there is no other implementation")


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe_{os.getpid()}_{threading.get_ident()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    env = os.environ.get("TQ_BUILD_DIR")
    if env:
        if not _writable_dir(env):
            raise KernelBuildError(f"$TQ_BUILD_DIR '{env}' cannot be written")
        return env
    local = os.path.join(_HERE, "_build")
    if _writable_dir(local):
        return local
    fallback = os.path.join(tempfile.gettempdir(), f"turboquant_cpp_b200_build_{os.getuid()}")
    if _writable_dir(fallback):
        return fallback
    raise KernelBuildError(f"neither '{local}' nor '{fallback}' can be written; set $TQ_BUILD_DIR")


def _source_hash(name: str, debug_index: Optional[bool] = None) -> str:
    h = hashlib.sha256()
    for fn in [name + ".cu"] + _HEADERS + [f for f in sorted(os.listdir(_HERE)) if f.endswith(".cuh")
                                           and f not in _HEADERS]:
        with open(os.path.join(_HERE, fn), "rb") as f:
            h.update(fn.encode())
            h.update(f.read())
    h.update(" ".join(_flags(name, debug_index)).encode())
    return h.hexdigest()[:16]


def library_path(name: str, debug_index: Optional[bool] = None) -> str:
    debug = DEBUG_INDEX if debug_index is None else debug_index
    return os.path.join(build_dir(), f"tq_{name}{'_checked' if debug else ''}_{_source_hash(name, debug)}.so")


def kernel_files() -> List[str]:
    return sorted(f[:-3] for f in os.listdir(_HERE) if f.endswith(".cu"))


def compile_kernel(name: str, verbose: bool = True, debug_index: Optional[bool] = None) -> str:
    """Builds one kernel file if its library is not there yet; returns the library's path."""
    src = os.path.join(_HERE, name + ".cu")
    if not os.path.isfile(src):
        raise KernelBuildError(f"no kernel file '{src}'")
    debug = DEBUG_INDEX if debug_index is None else debug_index
    out = library_path(name, debug)
    if os.path.isfile(out):
        return out
    nvcc = find_nvcc()
    tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [nvcc] + _flags(name, debug) + ["-I", _HERE, "-o", tmp, src]
    if verbose:
        _say(f"compiling {name}.cu for sm_100a{' with index checks' if debug else ''} …")
    t0 = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    # a line now and then while a long compile runs
    while True:
        try:
            log, _ = proc.communicate(timeout=20)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                _say(f"… still compiling {name}.cu ({time.time() - t0:.0f} s)")
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise KernelBuildError(f"nvcc failed on {name}.cu (exit {proc.returncode}):\n{log}")
    os.replace(tmp, out)
    prefix = f"tq_{name}{'_checked' if debug else ''}_"
    for old in os.listdir(os.path.dirname(out)):          # libraries of earlier versions of this file, same build
        stem = old[len(prefix):-3] if old.startswith(prefix) and old.endswith(".so") else ""
        if len(stem) == 16 and all(ch in "0123456789abcdef" for ch in stem) and os.path.join(os.path.dirname(out), old) != out:
            try:
                os.remove(os.path.join(os.path.dirname(out), old))
            except OSError:
                pass
    if verbose:
        _say(f"compiled {name}.cu in {time.time() - t0:.1f} s -> {out}")
    return out


def ensure_built(names: Iterable[str], verbose: bool = True, debug_index: Optional[bool] = None) -> None:
    """Builds several kernel files at once (one nvcc process each)."""
    own = debug_index is None or debug_index == DEBUG_INDEX
    names = [n for n in dict.fromkeys(names)
             if not (own and n in _loaded) and not os.path.isfile(library_path(n, debug_index))]
    if not names:
        return
    errors: List[BaseException] = []

    def work(n: str) -> None:
        try:
            compile_kernel(n, verbose, debug_index)
        except BaseException as e:  # noqa: BLE001 - reported below
            errors.append(e)

    threads = [threading.Thread(target=work, args=(n,)) for n in names]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise errors[0]


def load_kernel(name: str) -> ctypes.CDLL:
    """The loaded library of one kernel file, built first if needed."""
    with _lock:
        lib = _loaded.get(name)
        if lib is not None:
            return lib
        path = compile_kernel(name)
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelBuildError(f"cannot load '{path}': {e}") from None
        lib.tq_last_error.restype = ctypes.c_char_p
        _loaded[name] = lib
        return lib


INDEX_KINDS = {1: "a token id outside the vocabulary", 2: "a page id outside the cache", 3: "a position beyond the page table",
               4: "a sequence index outside the batch", 5: "an expert id outside the layer's experts",
               6: "a row outside the expert-sorted layout"}


def index_faults() -> List[str]:
    """What the index checks of the loaded libraries recorded since the last call (debug builds only; a release
    build records nothing).  Reading synchronises the device."""
    found = []
    for name, lib in list(_loaded.items()):
        rec = (ctypes.c_int * 4)()
        rc = lib.tq_index_fault_read(rec)
        if rc < 0:
            raise KernelBuildError(f"{name}: {lib.tq_last_error().decode('utf-8', 'replace')}")
        if rc == 1 and rec[0] != 0:
            found.append(f"{name}: {INDEX_KINDS.get(rec[0], f'index of kind {rec[0]}')}: {rec[1]} is not in "
                         f"0..{rec[2] - 1} (seen {rec[3]} time{'' if rec[3] == 1 else 's'} by the kernels' threads in all)")
    return found


def loaded_libraries() -> Dict[str, str]:
    return {n: l._name for n, l in _loaded.items()}
