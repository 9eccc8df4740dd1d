"""Builds the native modules and loads them with ctypes: the CUDA kernel modules for sm_100a
with nvcc, the host modules with the C++ compiler.

Each ``<name>.cu`` (kernels) or ``<name>.cpp`` (host code without CUDA) in this folder is one
module with ``extern "C"`` entry points; it is compiled to ``_build/lib<name>-<hash>.so``
where the hash covers the source, the shared headers and the compiler flags, so a stale
library is never loaded.  Modules are built on
demand: a model asks for the modules its parts need, and only those are compiled, in
parallel, with a progress line every few seconds.  There is no fallback: if nvcc is
missing or a module fails to build, loading raises :class:`KernelBuildError`.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import re
import tempfile
import threading
import time
from typing import Dict, Iterable, List, Optional

CSRC_DIR = os.path.dirname(os.path.abspath(__file__))

NVCC_FLAGS = [
    "-O3",
    "-std=c++17",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-shared",
    "-Xcompiler",
    "-fPIC",
]

# Flags of the host modules; $LOCUS_HOST_FLAGS adds to them (for instance "-fsanitize=address,undefined -g" for a
# checked build of the cache's and the scheduler's bookkeeping; the flags are part of the library's name).
HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-Wall"] + os.environ.get("LOCUS_HOST_FLAGS", "").split()

_INCLUDE = re.compile(r'^\s*#\s*include\s+"([^"]+)"', re.M)

# module name -> extra nvcc flags
MODULE_FLAGS: Dict[str, List[str]] = {}


class KernelBuildError(RuntimeError):
    pass


_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def _find_nvcc() -> str:
    for cand in (os.environ.get("LOCUS_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError(
        "nvcc not found (looked at $LOCUS_NVCC, PATH and /usr/local/cuda/bin): the CUDA "
        "kernels cannot be built and there is no fallback path"
    )


def _build_dir() -> str:
    d = os.environ.get("LOCUS_BUILD_DIR") or os.path.join(CSRC_DIR, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"locus_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _find_cxx() -> Optional[str]:
    for cand in (os.environ.get("CXX"), "g++", "c++", "clang++"):
        path = shutil.which(cand) if cand else None
        if path:
            return path
    return None


def module_names() -> List[str]:
    return sorted(os.path.splitext(f)[0] for f in os.listdir(CSRC_DIR) if f.endswith((".cu", ".cpp")))


def _is_host_module(name: str) -> bool:
    return os.path.isfile(os.path.join(CSRC_DIR, name + ".cpp"))


def source_files(name: str) -> List[str]:
    """The module's source file and every file of this folder that it includes with quotes, directly or through
    another one, in the order met: what a library's name is hashed over."""
    files = [name + (".cpp" if _is_host_module(name) else ".cu")]
    for f in files:  # grows while it is walked
        with open(os.path.join(CSRC_DIR, f), "r", encoding="utf-8") as fh:
            for inc in _INCLUDE.findall(fh.read()):
                if inc not in files and os.path.isfile(os.path.join(CSRC_DIR, inc)):
                    files.append(inc)
    return files


def _digest(name: str) -> str:
    h = hashlib.sha256()
    files = source_files(name)
    flags = HOST_FLAGS if _is_host_module(name) else NVCC_FLAGS + MODULE_FLAGS.get(name, [])
    for f in files:
        with open(os.path.join(CSRC_DIR, f), "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def library_path(name: str) -> str:
    return os.path.join(_build_dir(), f"lib{name}-{_digest(name)}.so")


def _compile_cmd(name: str, out: str) -> List[str]:
    if _is_host_module(name):
        src = os.path.join(CSRC_DIR, name + ".cpp")
        cxx = _find_cxx()
        if cxx is not None:
            return [cxx] + HOST_FLAGS + ["-o", out, src]
        # no C++ compiler of its own on the path: nvcc hands the file to the one it was set up with
        return [_find_nvcc(), "-O2", "-std=c++17", "-shared", "-Xcompiler", "-fPIC", "-o", out, src]
    return (
        [_find_nvcc()]
        + NVCC_FLAGS
        + MODULE_FLAGS.get(name, [])
        + ["-I", CSRC_DIR, "-o", out, os.path.join(CSRC_DIR, name + ".cu")]
    )


def build(names: Optional[Iterable[str]] = None, verbose: bool = True) -> Dict[str, str]:
    """Compile the named modules (default: all) that are not built yet; return their paths."""
    names = list(names) if names is not None else module_names()
    paths = {n: library_path(n) for n in names}
    todo = [n for n in names if not os.path.isfile(paths[n])]
    if not todo:
        return paths
    log = (lambda s: print(s, file=sys.stderr, flush=True)) if verbose else (lambda s: None)
    log(f"[locus_b200] compiling {len(todo)} module(s) (CUDA for sm_100a, host code): {', '.join(todo)}")
    procs = {}
    t0 = time.time()
    for n in todo:
        tmp = paths[n] + f".tmp{os.getpid()}"
        procs[n] = (
            subprocess.Popen(_compile_cmd(n, tmp), stdout=subprocess.PIPE, stderr=subprocess.STDOUT),
            tmp,
        )
    pending = set(todo)
    last = t0
    errors = []
    while pending:
        for n in list(pending):
            p, tmp = procs[n]
            if p.poll() is not None:
                out = p.stdout.read().decode(errors="replace")
                pending.discard(n)
                if p.returncode != 0:
                    errors.append(f"{n}:\n{out}")
                    if os.path.exists(tmp):
                        os.remove(tmp)
                else:
                    os.replace(tmp, paths[n])
                    # drop stale builds of the same module
                    d = os.path.dirname(paths[n])
                    for f in os.listdir(d):
                        if f.startswith(f"lib{n}-") and f.endswith(".so") and os.path.join(d, f) != paths[n]:
                            try:
                                os.remove(os.path.join(d, f))
                            except OSError:
                                pass
                    log(f"[locus_b200]   built {n} ({time.time() - t0:.0f}s)")
        if pending:
            time.sleep(0.2)
            if time.time() - last > 5.0:
                last = time.time()
                log(f"[locus_b200]   still compiling: {', '.join(sorted(pending))} ({last - t0:.0f}s)")
    if errors:
        raise KernelBuildError("compilation failed:\n" + "\n".join(errors))
    return paths


def load(name: str, verbose: bool = True) -> ctypes.CDLL:
    """The loaded library of module ``name``, compiling it first if needed."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = build([name], verbose=verbose)[name]
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelBuildError(f"cannot load kernel module {name}: {e}") from e
            _loaded[name] = lib
        return lib


def ensure(names: Iterable[str], verbose: bool = True) -> None:
    """Compile (in parallel) and load several modules at once."""
    names = [n for n in names if n not in _loaded]
    if names:
        build(names, verbose=verbose)
        for n in names:
            load(n, verbose=verbose)
