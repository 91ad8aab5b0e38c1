"""Loading the built kernel libraries and calling their C entry points."""

from __future__ import annotations

import ctypes
import threading
from typing import Dict

from . import build

_libs: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()
_launch_calls = 0          # kernels launched from Python (a captured graph replays them)


def launch_calls() -> int:
    return _launch_calls


def count_extra_launches(n: int = 1) -> None:
    """For entry points that launch more than one kernel (a merge kernel after the partial ones)."""
    global _launch_calls
    _launch_calls += n


class KernelError(RuntimeError):
    """A kernel launcher refused its arguments or CUDA reported an error."""


def library(module: str) -> ctypes.CDLL:
    with _lock:
        lib = _libs.get(module)
    if lib is None:
        path = build.ensure_built(module)
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load the CUDA kernel library {path}: {e}") from None
        with _lock:
            _libs[module] = lib
    return lib


def loaded_libraries() -> Dict[str, str]:
    with _lock:
        return {m: lib._name for m, lib in _libs.items()}


_cuda_error_names = {
    1: "invalid value", 2: "out of memory", 9: "invalid launch configuration",
    98: "invalid device function (library not built for this GPU)",
    209: "no kernel image for this device (the library is built for sm_100a only)",
    700: "illegal memory access", 715: "illegal instruction", 716: "misaligned address",
}


def check(status: int, what: str) -> None:
    if status == 0:
        return
    if status == -2:
        raise KernelError(f"{what}: a size or layout this kernel does not take")
    raise KernelError(f"{what}: CUDA error {status}"
                      f" ({_cuda_error_names.get(status, 'see cudaError_t')})")


class Function:
    """A C entry point with its argument types bound once."""

    def __init__(self, module: str, name: str, argtypes, check_status: bool = True):
        """``check_status`` False: the entry point launches nothing and returns a value, not a status."""
        self.module, self.name, self.argtypes = module, name, argtypes
        self.check_status = check_status
        self._fn = None

    def _bind(self):
        lib = library(self.module)
        try:
            fn = getattr(lib, self.name)
        except AttributeError:
            raise KernelError(f"{lib._name} has no entry point {self.name}") from None
        fn.argtypes = self.argtypes
        fn.restype = ctypes.c_int
        self._fn = fn
        return fn

    def __call__(self, *args):
        global _launch_calls
        fn = self._fn or self._bind()
        if not self.check_status:
            return fn(*args)
        _launch_calls += 1
        check(fn(*args), self.name)
