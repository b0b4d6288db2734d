"""Compiling and loading the native code.

Every native library is built from the sources in this folder at its first
use and cached under ``_build/`` beside them (or under the temporary folder
when the package folder cannot be written), keyed by a hash of the sources,
the headers and the flags.  CUDA sources are compiled by ``nvcc`` for sm_100a
only; host sources by ``g++``.  The libraries export plain C functions and are
loaded with :mod:`ctypes`.  There is no fallback: a library that cannot be
built or loaded raises :class:`~alofa_b200.errors.AlofaError` ("build")."""
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
from pathlib import Path

from ..errors import AlofaError

CSRC = Path(__file__).resolve().parent
NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-lineinfo", "-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
GXX_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-shared", "-Wall"]

_loaded: dict = {}
_lock = threading.Lock()
_load_lock = threading.RLock()


def _say(text: str) -> None:
    print(f"[alofa_b200] {text}", file=sys.stderr, flush=True)


_build_dir = None


def build_dir() -> Path:
    """Where compiled libraries are kept (decided once per process)."""
    global _build_dir
    with _lock:
        if _build_dir is None:
            _build_dir = _choose_build_dir()
        return _build_dir


def _choose_build_dir() -> Path:
    override = os.environ.get("ALOFA_BUILD_DIR")
    candidates = [Path(override)] if override else []
    candidates += [CSRC / "_build", Path(tempfile.gettempdir()) / f"alofa_b200_build_{os.getuid()}"]
    for cand in candidates:
        try:
            cand.mkdir(parents=True, exist_ok=True)
            probe = cand / f".probe{os.getpid()}"
            probe.write_text("")
            probe.unlink()
            return cand
        except OSError:
            continue
    raise AlofaError("build", "no writable folder for compiled libraries", f"tried={[str(c) for c in candidates]}")


def _find(tool: str, extra: list) -> str:
    for cand in extra:
        if cand and Path(cand).exists():
            return str(cand)
    found = shutil.which(tool)
    if found:
        return found
    raise AlofaError("build", f"{tool} was not found", "needed to compile the native code of alofa_b200")


def _nvcc() -> str:
    home = os.environ.get("CUDA_HOME") or os.environ.get("CUDA_PATH")
    return _find("nvcc", [f"{home}/bin/nvcc" if home else None, "/usr/local/cuda/bin/nvcc"])


def _key(sources: list, defines: dict, flags: list) -> str:
    h = hashlib.sha256()
    for src in sources:
        h.update(Path(src).read_bytes())
    for header in sorted(CSRC.rglob("*.cuh")) + sorted(CSRC.rglob("*.h")):
        h.update(header.read_bytes())
    h.update(repr(sorted(defines.items())).encode())
    h.update(repr(flags).encode())
    return h.hexdigest()[:16]


def library_path(name: str, sources: list, defines: dict | None = None, cuda: bool = True, extra_flags: list | None = None) -> tuple:
    defines = defines or {}
    flags = (NVCC_ARCH + NVCC_FLAGS if cuda else GXX_FLAGS) + (extra_flags or [])
    srcs = [str(CSRC / s) for s in sources]
    key = _key(srcs, defines, flags)
    return build_dir() / f"{name}-{key}.so", srcs, flags


def compile_library(name: str, sources: list, defines: dict | None = None, cuda: bool = True, extra_flags: list | None = None) -> Path:
    """Build the library if its cached copy is missing; return its path."""
    defines = defines or {}
    out, srcs, flags = library_path(name, sources, defines, cuda, extra_flags)
    if out.exists():
        return out
    tmp = out.with_suffix(f".tmp{os.getpid()}.so")
    dflags = [f"-D{k}={v}" for k, v in sorted(defines.items())]
    if cuda:
        cmd = [_nvcc()] + flags + dflags + ["-I", str(CSRC), "-o", str(tmp)] + srcs
    else:
        cmd = [_find("g++", [])] + flags + dflags + ["-I", str(CSRC), "-o", str(tmp)] + srcs
    _say(f"compiling {name} ({'sm_100a' if cuda else 'host'}) ...")
    start = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    done = threading.Event()

    def heartbeat():
        while not done.wait(10.0):
            _say(f"still compiling {name} ({time.time() - start:.0f} s) ...")

    beat = threading.Thread(target=heartbeat, daemon=True)
    beat.start()
    output, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        if tmp.exists():
            tmp.unlink()
        raise AlofaError("build", f"compiling {name} failed", f"command={' '.join(cmd)}\n{output}")
    os.replace(tmp, out)
    for stale in out.parent.glob(f"{name}-*.so"):  # older builds of the same library
        if stale != out and ".tmp" not in stale.name:
            try:
                stale.unlink()
            except OSError:
                pass
    _say(f"compiled {name} in {time.time() - start:.1f} s")
    return out


def load_library(name: str, sources: list, defines: dict | None = None, cuda: bool = True, extra_flags: list | None = None) -> ctypes.CDLL:
    """The loaded library, compiling it first when needed."""
    ident = (name, tuple(sources), tuple(sorted((defines or {}).items())), cuda, tuple(extra_flags or []))
    with _load_lock:
        if ident in _loaded:
            return _loaded[ident]
        path = compile_library(name, sources, defines, cuda, extra_flags)
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as err:
            raise AlofaError("build", f"loading {name} failed", f"path={path}: {err}") from err
        _loaded[ident] = lib
        return lib


def compile_many(jobs: list, workers: int = 0) -> list:
    """Compile several libraries side by side; ``jobs`` are keyword dicts of
    :func:`compile_library`."""
    from concurrent.futures import ThreadPoolExecutor

    workers = workers or min(len(jobs), os.cpu_count() or 4) or 1
    with ThreadPoolExecutor(max_workers=workers) as pool:
        return list(pool.map(lambda kw: compile_library(**kw), jobs))
