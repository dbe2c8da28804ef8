"""Compiling the CUDA sources of ``csrc/`` for sm_100a and loading them.

Each module (one ``.cu`` file plus a set of ``-D`` definitions) becomes one shared
object with a plain C interface, loaded with ``ctypes``.  Objects are built at
first use, next to the sources under ``csrc/_build/`` when that folder can be
written, else under ``$FIREFLY_B200_BUILD_DIR`` or a per-user folder in the
temporary directory.  The file name carries a hash of the sources and flags, so
a changed kernel is rebuilt and a stale object is never loaded.  While ``nvcc``
runs, a line is printed to stderr every few seconds.

There is no fallback: if ``nvcc`` is missing or the compilation fails, the call
raises ``KernelBuildError``.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import Dict, Iterable, Mapping, Optional, Sequence, Tuple

CSRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr", "-Xcudafe", "--diag_suppress=177"]


class KernelBuildError(RuntimeError):
    pass


_loaded: Dict[tuple, ctypes.CDLL] = {}
_lock = threading.Lock()


def find_nvcc() -> str:
    for cand in (os.environ.get("FIREFLY_B200_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError("nvcc not found (looked at $FIREFLY_B200_NVCC, $CUDA_HOME/bin, PATH, "
                           "/usr/local/cuda/bin); the CUDA kernels cannot be built and there is no "
                           "other implementation")


_build_dir: Optional[str] = None
_build_dir_lock = threading.Lock()


def build_dir() -> str:
    """The folder objects are built into (chosen once per process)."""
    global _build_dir
    with _build_dir_lock:
        if _build_dir is not None:
            return _build_dir
        cands = []
        if os.environ.get("FIREFLY_B200_BUILD_DIR"):
            cands.append(os.environ["FIREFLY_B200_BUILD_DIR"])
        cands.append(os.path.join(CSRC, "_build"))
        cands.append(os.path.join(tempfile.gettempdir(), f"firefly_b200-build-{os.getuid()}"))
        for d in cands:
            try:
                os.makedirs(d, exist_ok=True)
                fd, probe = tempfile.mkstemp(prefix=".probe", dir=d)
                os.close(fd)
                os.unlink(probe)
                _build_dir = d
                return d
            except OSError:
                continue
        raise KernelBuildError(f"no writable build folder among {cands}")


def _hash(paths: Iterable[str], flags: Sequence[str]) -> str:
    h = hashlib.sha1()
    for p in sorted(paths):
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:12]


def _headers() -> Sequence[str]:
    return [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith((".cuh", ".h"))]


def _included_sources(src: str) -> Sequence[str]:
    """Files of ``csrc/`` that ``src`` pulls in with ``#include "..."``, followed through (a module may
    include another module's ``.cu`` to share its kernels); they are part of what the object is made of."""
    seen, todo = [], [src]
    while todo:
        path = todo.pop()
        try:
            with open(path, "r", encoding="utf-8", errors="replace") as fh:
                lines = fh.read().splitlines()
        except OSError:
            continue
        for line in lines:
            line = line.strip()
            if line.startswith("#include \""):
                inc = os.path.join(CSRC, line.split('"')[1])
                if os.path.isfile(inc) and inc not in seen and inc != src:
                    seen.append(inc)
                    todo.append(inc)
    return seen


def library_path(source: str, defines: Optional[Mapping[str, object]] = None) -> Tuple[str, Sequence[str]]:
    src = os.path.join(CSRC, source)
    if not os.path.isfile(src):
        raise KernelBuildError(f"kernel source missing: {src}")
    dflags = [f"-D{k}={v}" for k, v in sorted((defines or {}).items())]
    flags = ARCH_FLAGS + BASE_FLAGS + dflags
    tag = _hash(sorted({src, *_headers(), *_included_sources(src)}), flags)
    stem = os.path.splitext(source)[0]
    suffix = "".join(f"_{k.lower()}{v}" for k, v in sorted((defines or {}).items()))
    return os.path.join(build_dir(), f"ff_{stem}{suffix}-{tag}.so"), flags


def compile_module(source: str, defines: Optional[Mapping[str, object]] = None, *,
                   verbose: bool = True) -> str:
    """Build (if needed) and return the path of the module's shared object."""
    out, flags = library_path(source, defines)
    if os.path.isfile(out):
        return out
    nvcc = find_nvcc()
    src = os.path.join(CSRC, source)
    lock_path = out + ".lock"
    with open(lock_path, "w") as lock_fh:
        fcntl.flock(lock_fh, fcntl.LOCK_EX)
        try:
            if os.path.isfile(out):
                return out
            tmp = f"{out}.tmp{os.getpid()}"
            cmd = [nvcc, *flags, "-I", CSRC, "-o", tmp, src]
            t0 = time.time()
            if verbose:
                print(f"[firefly_b200] compiling {os.path.basename(out)} for sm_100a ...",
                      file=sys.stderr, flush=True)
            proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            done = threading.Event()

            def _tick():
                while not done.wait(8.0):
                    if verbose:
                        print(f"[firefly_b200]   still compiling {source} ({time.time() - t0:.0f} s)",
                              file=sys.stderr, flush=True)
            ticker = threading.Thread(target=_tick, daemon=True)
            ticker.start()
            log, _ = proc.communicate()
            done.set()
            if proc.returncode != 0 or not os.path.isfile(tmp):
                raise KernelBuildError(f"nvcc failed for {source} (exit {proc.returncode}):\n"
                                       f"{' '.join(cmd)}\n{log}")
            os.replace(tmp, out)
            # objects of the same module built from older sources are of no use any more
            stem = os.path.basename(out).rsplit("-", 1)[0]
            for f in os.listdir(os.path.dirname(out)):
                if f.endswith(".so") and f.rsplit("-", 1)[0] == stem and f != os.path.basename(out):
                    try:
                        os.unlink(os.path.join(os.path.dirname(out), f))
                    except OSError:
                        pass
            if verbose:
                print(f"[firefly_b200] built {os.path.basename(out)} in {time.time() - t0:.1f} s",
                      file=sys.stderr, flush=True)
        finally:
            fcntl.flock(lock_fh, fcntl.LOCK_UN)
    try:
        os.unlink(lock_path)
    except OSError:
        pass
    return out


def find_cxx() -> str:
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")):
        if cand and shutil.which(cand):
            return shutil.which(cand)
    raise KernelBuildError("no C++ compiler found (looked at $CXX, g++, c++, clang++)")


def load_host_module(source: str) -> ctypes.CDLL:
    """Build (with the host C++ compiler) and load a host-only module of ``csrc/``."""
    key = ("host", source)
    lib = _loaded.get(key)
    if lib is not None:
        return lib
    with _lock:
        lib = _loaded.get(key)
        if lib is not None:
            return lib
        src = os.path.join(CSRC, source)
        if not os.path.isfile(src):
            raise KernelBuildError(f"source missing: {src}")
        flags = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden"]
        tag = _hash([src], flags)
        stem = os.path.splitext(os.path.basename(source))[0]
        out = os.path.join(build_dir(), f"ffh_{stem}-{tag}.so")
        if not os.path.isfile(out):
            with open(out + ".lock", "w") as lock_fh:
                fcntl.flock(lock_fh, fcntl.LOCK_EX)
                try:
                    if not os.path.isfile(out):
                        tmp = f"{out}.tmp{os.getpid()}"
                        cmd = [find_cxx(), *flags, "-o", tmp, src]
                        proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
                        if proc.returncode != 0 or not os.path.isfile(tmp):
                            raise KernelBuildError(f"C++ build failed for {source}:\n{' '.join(cmd)}\n{proc.stdout}")
                        os.replace(tmp, out)
                        for f in os.listdir(os.path.dirname(out)):
                            if f.startswith(f"ffh_{stem}-") and f.endswith(".so") and f != os.path.basename(out):
                                try:
                                    os.unlink(os.path.join(os.path.dirname(out), f))
                                except OSError:
                                    pass
                finally:
                    fcntl.flock(lock_fh, fcntl.LOCK_UN)
            try:
                os.unlink(out + ".lock")
            except OSError:
                pass
        try:
            lib = ctypes.CDLL(out)
        except OSError as e:
            raise KernelBuildError(f"cannot load {out}: {e}") from e
        _loaded[key] = lib
    return lib


def load_module(source: str, defines: Optional[Mapping[str, object]] = None) -> ctypes.CDLL:
    key = (source, tuple(sorted((defines or {}).items())))
    lib = _loaded.get(key)
    if lib is not None:
        return lib
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            path = compile_module(source, defines)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from e
            _loaded[key] = lib
    return lib


def compile_many(modules: Sequence[Tuple[str, Optional[Mapping[str, object]]]]) -> None:
    """Build several modules at once (one nvcc process each, in parallel)."""
    errors = []

    def _one(src, defs):
        try:
            compile_module(src, defs)
        except Exception as e:  # noqa: BLE001 - reported below
            errors.append(e)
    threads = [threading.Thread(target=_one, args=m) for m in modules]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise errors[0]
