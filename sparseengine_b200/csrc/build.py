"""Compile the CUDA sources of this folder for sm_100a, each into a shared library of its own.

There is no install step.  Every source is self-contained (the sources share headers, no
symbols), so a launcher's source is compiled into ``_build/`` beside the sources the first time
the launcher is used, and later runs find the library by the hash of its source, the headers
and the flags: a program compiles the kernels its model needs and no more.  ``build()`` compiles
all of them at once, in parallel (well under a minute; the sources use no framework headers).
If the package folder is not writable the build goes to a per-user folder under the system's
temporary directory.  There is no fallback: if a library cannot be built or loaded, the op that
needs it raises.
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
from concurrent.futures import ThreadPoolExecutor, as_completed

_HERE = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH_FLAGS + ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr",
                           "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default"]
NVCC_FLAGS += os.environ.get("SPARSEENGINE_NVCC_FLAGS", "").split()     # e.g. -D switches for experiments

_lock = threading.Lock()
_lib = None


def _say(msg: str) -> None:
    print(f"[sparseengine_b200] {msg}", file=sys.stderr, flush=True)


def sources() -> list[str]:
    return sorted(f for f in os.listdir(_HERE) if f.endswith(".cu"))


def _headers_digest() -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(_HERE)):
        if f.endswith((".cuh", ".h")):
            with open(os.path.join(_HERE, f), "rb") as fh:
                h.update(f.encode() + b"\0" + fh.read())
    return h.hexdigest()


def find_nvcc() -> str:
    for cand in (os.environ.get("SPARSEENGINE_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise RuntimeError("nvcc not found (set CUDA_HOME or SPARSEENGINE_NVCC); the CUDA kernels "
                       "of sparseengine_b200 have to be compiled and there is no fallback")


def build_dir() -> str:
    want = os.environ.get("SPARSEENGINE_BUILD_DIR") or os.path.join(_HERE, "_build")
    try:
        os.makedirs(want, exist_ok=True)
        probe = os.path.join(want, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return want
    except OSError:
        alt = os.path.join(tempfile.gettempdir(), f"sparseengine_b200_build_{os.getuid()}")
        os.makedirs(alt, exist_ok=True)
        return alt


def _library_name(src: str, hdr: str) -> str:
    with open(os.path.join(_HERE, src), "rb") as f:
        digest = hashlib.sha256(f.read() + hdr.encode() + " ".join(NVCC_FLAGS).encode()).hexdigest()[:16]
    return f"{os.path.splitext(src)[0]}.{digest}.so"


_EXPORT = re.compile(r'extern\s+"C"\s+[\w\s\*]*?\b(se_\w+)\s*\(')
_exports = None


def exports() -> dict:
    """Exported launcher name -> the source file that defines it (read from the sources' text)."""
    global _exports
    if _exports is None:
        found = {}
        for src in sources():
            with open(os.path.join(_HERE, src)) as f:
                for name in _EXPORT.findall(f.read()):
                    found[name] = src
        _exports = found
    return _exports


def _compile_one(nvcc: str, src: str, lib: str) -> None:
    tmp = f"{lib}.tmp{os.getpid()}"
    cmd = [nvcc, *NVCC_FLAGS, "-I", _HERE, "-shared", os.path.join(_HERE, src), "-o", tmp]
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    r = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)


def _drop_older(out: str, src: str, keep: str) -> None:
    stem = os.path.splitext(src)[0] + "."
    for f in os.listdir(out):
        if f.startswith(stem) and f.endswith((".so", ".o")) and os.path.join(out, f) != keep:
            try:
                os.remove(os.path.join(out, f))
            except OSError:
                pass


def build_source(src: str, verbose: bool = True) -> str:
    """Compile one source into a shared library of its own, if it is stale; return its path."""
    out = build_dir()
    lib = os.path.join(out, _library_name(src, _headers_digest()))
    if not os.path.isfile(lib):
        t0 = time.time()
        if verbose:
            _say(f"compiling {src} for sm_100a into {out} (first use only)")
        _compile_one(find_nvcc(), src, lib)
        _drop_older(out, src, lib)
        if verbose:
            _say(f"  compiled {src} ({time.time() - t0:.0f}s)")
    return lib


def build(verbose: bool = True) -> list:
    """Compile every stale source (in parallel), each into its own shared library; return the
    libraries' paths.  Nothing needs this call: a launcher's library is compiled when the launcher is
    first used, so a program compiles what its model needs and no more."""
    out = build_dir()
    hdr = _headers_digest()
    srcs = sources()
    libs = [os.path.join(out, _library_name(s, hdr)) for s in srcs]
    stale = [(s, o) for s, o in zip(srcs, libs) if not os.path.isfile(o)]
    if stale:
        nvcc = find_nvcc()
        t0 = time.time()
        if verbose:
            _say(f"compiling {len(stale)} CUDA source(s) for sm_100a into {out}")
        with ThreadPoolExecutor(max_workers=min(len(stale), os.cpu_count() or 4)) as pool:
            futs = {pool.submit(_compile_one, nvcc, s, o): (s, o) for s, o in stale}
            for done, f in enumerate(as_completed(futs), 1):
                f.result()
                s, o = futs[f]
                _drop_older(out, s, o)
                if verbose:
                    _say(f"  compiled {s} ({done}/{len(stale)}, {time.time() - t0:.0f}s)")
    return libs


class Library:
    """The launchers of all sources as attributes; a source is compiled (if stale) and loaded when
    one of its launchers is first asked for."""

    def __init__(self):
        self._loaded = {}

    def __getattr__(self, name: str):
        if name.startswith("_"):
            raise AttributeError(name)
        src = exports().get(name)
        if src is None:
            raise AttributeError(f"no CUDA source of sparseengine_b200 exports {name!r}")
        with _lock:
            lib = self._loaded.get(src)
            if lib is None:
                lib = self._loaded[src] = ctypes.CDLL(build_source(src), mode=ctypes.RTLD_LOCAL)
        fn = getattr(lib, name)
        self.__dict__[name] = fn
        return fn

    def loaded_sources(self) -> list:
        return sorted(self._loaded)


def load() -> Library:
    """The library object (once per process).  It compiles nothing by itself."""
    global _lib
    if _lib is None:
        _lib = Library()
    return _lib
