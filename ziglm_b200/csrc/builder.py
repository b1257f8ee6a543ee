"""Compiles the CUDA sources of this folder for sm_100a and loads them with ctypes.

Each ``<name>.cu`` becomes one shared library ``_build/<name>-<hash>.so`` beside the
sources (the hash covers the source, the shared headers and the flags, so an
edited file is rebuilt and an unchanged one is loaded as it is).  A library is
built the first time something asks for it, so a model compiles what its parts
need and nothing else.  Building prints a line when it starts, every few seconds
while it runs, and when it ends.

The reference compiles its one CUDA file with ``nvcc -O3 -Xcompiler -fPIC`` for
sm_75..sm_90 (build.zig:39-76) and links it into the host program; here the
target is sm_100a only and the host binds through the C ABI at run time.
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
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, Iterable, List, Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
_HEADERS = ("common.cuh", "tc_common.cuh", "attention_noalloc.h")
_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--shared",
]
_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}


class KernelBuildError(RuntimeError):
    """A CUDA source could not be compiled or its library could not be loaded."""


def sources() -> List[str]:
    """Names (without .cu) of every CUDA source of the library."""
    return sorted(f[:-3] for f in os.listdir(_HERE) if f.endswith(".cu"))


def _nvcc() -> str:
    for cand in (os.environ.get("ZIGLM_B200_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise KernelBuildError("nvcc was not found (set ZIGLM_B200_NVCC or CUDA_HOME); the CUDA kernels of this "
                           "library are compiled at first use and there is no other path")


_dir: Optional[str] = None


def _build_dir() -> str:
    """Where libraries are kept: beside the sources, or a per-user temporary folder if that is read-only."""
    global _dir
    with _lock:
        if _dir is not None:
            return _dir
        d = os.environ.get("ZIGLM_B200_BUILD_DIR") or os.path.join(_HERE, "_build")
        try:
            os.makedirs(d, exist_ok=True)
            fd, probe = tempfile.mkstemp(prefix=".w", dir=d)
            os.close(fd)
            os.unlink(probe)
        except OSError:
            d = os.path.join(tempfile.gettempdir(), f"ziglm_b200_build_{os.getuid()}")
            os.makedirs(d, exist_ok=True)
        _dir = d
        return d


def _digest(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(_FLAGS).encode())
    for f in (name + ".cu",) + _HEADERS:
        p = os.path.join(_HERE, f)
        if os.path.exists(p):
            with open(p, "rb") as fh:
                h.update(fh.read())
    return h.hexdigest()[:16]


def library_path(name: str) -> str:
    return os.path.join(_build_dir(), f"{name}-{_digest(name)}.so")


def _say(msg: str) -> None:
    print(f"[ziglm_b200] {msg}", file=sys.stderr, flush=True)


def _compile(name: str) -> str:
    src = os.path.join(_HERE, name + ".cu")
    if not os.path.exists(src):
        raise KernelBuildError(f"no CUDA source {name}.cu in {_HERE}")
    out = library_path(name)
    if os.path.exists(out):
        return out
    nvcc = _nvcc()
    tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [nvcc] + _FLAGS + ["-I", _HERE, "-o", tmp, src]
    _say(f"compiling {name}.cu for sm_100a ...")
    t0 = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env, cwd=_HERE)
    done = threading.Event()

    def heartbeat() -> None:
        while not done.wait(10.0):
            _say(f"still compiling {name}.cu ({time.time() - t0:.0f} s)")

    hb = threading.Thread(target=heartbeat, daemon=True)
    hb.start()
    try:
        log, _ = proc.communicate()
    finally:
        done.set()
    if proc.returncode != 0:
        try:
            os.unlink(tmp)
        except OSError:
            pass
        raise KernelBuildError(f"nvcc failed on {name}.cu (exit {proc.returncode}):\n{log.decode(errors='replace')}")
    os.replace(tmp, out)
    # older builds of the same source are of no use any more
    prefix = name + "-"
    for f in os.listdir(os.path.dirname(out)):
        if f.startswith(prefix) and f.endswith(".so") and os.path.join(os.path.dirname(out), f) != out:
            try:
                os.unlink(os.path.join(os.path.dirname(out), f))
            except OSError:
                pass
    _say(f"compiled {name}.cu in {time.time() - t0:.1f} s")
    return out


def build(names: Optional[Iterable[str]] = None, jobs: Optional[int] = None) -> List[str]:
    """Compile the named sources (all of them by default), several at a time."""
    todo = list(names) if names is not None else sources()
    jobs = jobs or min(len(todo), max(1, (os.cpu_count() or 2)))
    if not todo:
        return []
    with ThreadPoolExecutor(max_workers=jobs) as pool:
        return list(pool.map(_compile, todo))


def is_loaded(name: str) -> bool:
    with _lock:
        return name in _loaded


def load(name: str) -> ctypes.CDLL:
    """The shared library of ``<name>.cu``, compiled first if need be."""
    with _lock:
        lib = _loaded.get(name)
        if lib is not None:
            return lib
    path = _compile(name)
    try:
        lib = ctypes.CDLL(path)
    except OSError as e:
        raise KernelBuildError(f"could not load {path}: {e}") from None
    with _lock:
        _loaded.setdefault(name, lib)
        return _loaded[name]
