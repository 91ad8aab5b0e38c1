"""Loading the built kernel libraries and calling their C entry points."""

from __future__ import annotations

import ctypes
import threading
from typing import Dict

from . import build

_libs: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()
_launch_calls = 0          # kernels launched from Python (a captured graph replays them)
_recorder = None           # the list of the active LaunchRecord
_pending_cost = None       # what the launcher said about the launch that comes next


def launch_calls() -> int:
    return _launch_calls


def count_extra_launches(n: int = 1) -> None:
    """For entry points that launch more than one kernel (a merge kernel after the partial ones)."""
    global _launch_calls
    _launch_calls += n


class LaunchRecord:
    """Collects every launch made while it is active, so that the same launches (same pointers,
    same sizes) can be issued again, alone or grouped by entry point, for timing.

    An entry is ``(name, issue, cost)``: ``issue(stream)`` launches it again on the raw stream
    handle ``stream`` and ``cost`` is what the launcher said the launch has to move and compute,
    ``{"bytes": ..., "flops": ...}`` (see :func:`annotate`; empty if it said nothing).  The
    tensors behind the recorded pointers must outlive the record."""

    def __init__(self):
        self.launches = []

    def __enter__(self):
        global _recorder
        if _recorder is not None:
            raise RuntimeError("a launch record is already active")
        _recorder = self.launches
        return self

    def __exit__(self, *exc):
        global _recorder, _pending_cost
        _recorder = None
        _pending_cost = None
        return False

    def names(self):
        """Entry points in the order of their first launch."""
        seen = []
        for name, _, _ in self.launches:
            if name not in seen:
                seen.append(name)
        return seen

    def cost(self, name: str = None):
        """Summed bytes and flops of the recorded launches (of ``name`` only, if given)."""
        total = {"bytes": 0, "flops": 0, "launches": 0}
        for n, _, c in self.launches:
            if name is None or n == name:
                total["bytes"] += c.get("bytes", 0)
                total["flops"] += c.get("flops", 0)
                total["launches"] += 1
        return total

    def issue(self, stream: int, name: str = None) -> int:
        """Launch again, on ``stream`` (a raw handle), every recorded launch (of entry point
        ``name`` only, if given); returns how many."""
        n = 0
        for launch_name, again, _ in self.launches:
            if name is None or launch_name == name:
                again(stream)
                n += 1
        return n


def recording() -> bool:
    return _recorder is not None


def annotate(bytes: int = 0, flops: int = 0, label: str = "") -> None:
    """Called by a launcher just before its launch while a record is active: the bytes the
    launch has to read and write and the floating-point operations it has to do.  ``label``
    (a shape, say) tells launches of one entry point apart in the record: the entry is named
    ``entry_point[label]``."""
    global _pending_cost
    _pending_cost = {"bytes": int(bytes), "flops": int(flops), "label": label}


def record_library_call(name: str, again, bytes: int = 0, flops: int = 0) -> None:
    """Put a library call (a cuBLAS product through torch) into the active record; ``again()``
    repeats it on torch's current stream."""
    if _recorder is not None:
        _recorder.append((name, lambda stream: again(), {"bytes": int(bytes), "flops": int(flops)}))


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
        if _recorder is not None:
            global _pending_cost
            head, cost, _pending_cost = args[:-1], _pending_cost or {}, None
            name = f"{self.name}[{cost['label']}]" if cost.get("label") else self.name
            _recorder.append((name, lambda stream: check(fn(*head, stream), self.name), cost))
        check(fn(*args), self.name)
