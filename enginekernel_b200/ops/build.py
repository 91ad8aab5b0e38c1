"""Compiling the CUDA sources for sm_100a and finding the built libraries.

Each ``csrc/<module>.cu`` becomes one shared library ``ek_<module>.<hash>.so`` with
plain C entry points (no Python or torch headers, so a module compiles in seconds).
The hash covers the source, the shared header and the compiler flags: a stale library
is never loaded.  Libraries are built on first use of a module - a model compiles only
what it needs - into ``enginekernel_b200/_build`` when that folder can be written, else
into a per-user folder under the system's temporary directory (or ``EK_B200_BUILD_DIR``).
Nothing is read from or written to the home directory.  The reference has no build step
(its kernels are JIT-compiled by Triton; engine/engine.py:28-44 only makes Triton's cache
folder writable).
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, Iterable, List

CSRC = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc")
CSRC = os.path.normpath(CSRC)

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "--shared", "-Xcompiler", "-fPIC,-fvisibility=hidden"]

_lock = threading.Lock()
_built: Dict[str, str] = {}


class BuildError(RuntimeError):
    pass


def modules() -> List[str]:
    return sorted(f[:-3] for f in os.listdir(CSRC) if f.endswith(".cu"))


def _nvcc() -> str:
    for cand in (os.environ.get("EK_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc was not found (looked at EK_B200_NVCC, PATH and /usr/local/cuda/bin); "
                     "the CUDA kernels of enginekernel_b200 cannot be built")


def _writable(folder: str) -> bool:
    try:
        os.makedirs(folder, exist_ok=True)
        with tempfile.NamedTemporaryFile(dir=folder):
            pass
        return True
    except OSError:
        return False


def build_dir() -> str:
    env = os.environ.get("EK_B200_BUILD_DIR")
    if env:
        if not _writable(env):
            raise BuildError(f"EK_B200_BUILD_DIR={env} cannot be written")
        return env
    in_tree = os.path.normpath(os.path.join(CSRC, "..", "_build"))
    if _writable(in_tree):
        return in_tree
    uid = os.getuid() if hasattr(os, "getuid") else 0
    out = os.path.join(tempfile.gettempdir(), f"enginekernel_b200_build_{uid}")
    if not _writable(out):
        raise BuildError(f"no writable folder for built kernels (tried {in_tree} and {out}); "
                         "set EK_B200_BUILD_DIR")
    return out


def _digest(module: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for name in sorted(os.listdir(CSRC)):
        if name == module + ".cu" or name.endswith(".cuh"):
            with open(os.path.join(CSRC, name), "rb") as f:
                h.update(name.encode())
                h.update(f.read())
    return h.hexdigest()[:16]


def library_path(module: str) -> str:
    return os.path.join(build_dir(), f"ek_{module}.{_digest(module)}.so")


def _say(msg: str) -> None:
    print(f"[enginekernel_b200] {msg}", file=sys.stderr, flush=True)


def _compile(module: str, out: str) -> None:
    src = os.path.join(CSRC, module + ".cu")
    if not os.path.exists(src):
        raise BuildError(f"no kernel source {src}")
    folder = os.path.dirname(out)
    fd, tmp = tempfile.mkstemp(prefix=f"ek_{module}.", suffix=".so.tmp", dir=folder)
    os.close(fd)
    cmd = [_nvcc()] + NVCC_FLAGS + ["-I", CSRC, "-o", tmp, src]
    _say(f"compiling {module}.cu for sm_100a")
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                            cwd=folder)
    try:
        while True:
            try:
                log, _ = proc.communicate(timeout=15)
                break
            except subprocess.TimeoutExpired:
                _say(f"still compiling {module}.cu ({time.time() - t0:.0f} s)")
        if proc.returncode != 0:
            raise BuildError(f"nvcc failed on {module}.cu:\n{log}")
        os.replace(tmp, out)
    finally:
        if os.path.exists(tmp):
            os.unlink(tmp)
    # drop libraries of older versions of this module
    prefix = f"ek_{module}."
    for name in os.listdir(folder):
        if name.startswith(prefix) and name.endswith(".so") and os.path.join(folder, name) != out:
            try:
                os.unlink(os.path.join(folder, name))
            except OSError:
                pass
    _say(f"built {os.path.basename(out)} in {time.time() - t0:.1f} s")


def ensure_built(module: str) -> str:
    """Path of the up-to-date library of ``module``, compiling it if needed."""
    with _lock:
        if module in _built:
            return _built[module]
    out = library_path(module)
    if not os.path.exists(out):
        _compile(module, out)
    with _lock:
        _built[module] = out
    return out


def build_all(names: Iterable[str] = None, jobs: int = None) -> Dict[str, str]:
    """Compile every module (or ``names``) in parallel; returns module -> library path."""
    names = list(names) if names is not None else modules()
    jobs = jobs or min(len(names), os.cpu_count() or 1) or 1
    with ThreadPoolExecutor(max_workers=jobs) as pool:
        paths = list(pool.map(ensure_built, names))
    return dict(zip(names, paths))
