"""Loading the compiled kernel libraries and calling their exported C functions.

There is no other implementation behind these calls: if a library cannot be built or loaded,
or a function reports an error, a ``KernelError`` is raised.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Dict

from ..csrc import build as _build


class KernelError(RuntimeError):
    """A kernel library is missing, or one of its functions refused its arguments."""


_lock = threading.Lock()
_loaded: Dict[str, "KernelLibrary"] = {}
_observer = None


def set_call_observer(fn) -> None:
    """``fn(function name, "begin" | "end")`` is called around every exported function that
    launches (None: nobody watches).  The benchmark uses it to put CUDA events around each kernel
    of one instrumented step; nothing on the product path sets it."""
    global _observer
    _observer = fn


class KernelLibrary:
    def __init__(self, name: str):
        try:
            self.path = _build.library_path(name)
        except _build.BuildError as e:
            raise KernelError(f"kernel library '{name}' is not available: {e}") from e
        try:
            self.lib = ctypes.CDLL(self.path)
        except OSError as e:
            raise KernelError(f"kernel library '{name}' ({self.path}) cannot be loaded: {e}") from e
        self.name = name
        self.lib.bfi_last_error.restype = ctypes.c_char_p
        self._funcs: Dict[str, ctypes._CFuncPtr] = {}
        self.calls = 0          # exported functions called so far (each launches at least one kernel)
        # Programmatic dependent launch is on: a kernel may start, and stream weights into its
        # shared memory, while its predecessor still runs.  BFI_B200_PDL=0 turns it off.
        if os.environ.get("BFI_B200_PDL", "1") == "0":
            self.lib.bfi_set_pdl(ctypes.c_int(0))

    def call_optional(self, func: str, *args) -> bool:
        """For kernels that may decline a shape: True if it ran, False if it declined (code 2)."""
        f = self._function(func)
        if _observer is not None:
            _observer(func, "begin")
        rc = f(*args)
        if _observer is not None:
            _observer(func, "end" if rc != 2 else "declined")
        if rc == 2:
            return False
        self.calls += 1
        if rc != 0:
            raise KernelError(self.lib.bfi_last_error().decode("utf-8", "replace"))
        return True

    def _function(self, func: str):
        f = self._funcs.get(func)
        if f is None:
            try:
                f = getattr(self.lib, func)
            except AttributeError as e:
                raise KernelError(f"kernel library '{self.name}' has no function {func}") from e
            f.restype = ctypes.c_int
            self._funcs[func] = f
        return f

    def call(self, func: str, *args) -> None:
        f = self._funcs.get(func)
        if f is None:
            try:
                f = getattr(self.lib, func)
            except AttributeError as e:
                raise KernelError(f"kernel library '{self.name}' has no function {func}") from e
            f.restype = ctypes.c_int
            self._funcs[func] = f
        self.calls += 1
        if _observer is not None:
            _observer(func, "begin")
        rc = f(*args)
        if _observer is not None:
            _observer(func, "end")
        if rc != 0:
            raise KernelError(self.lib.bfi_last_error().decode("utf-8", "replace"))


def total_calls() -> int:
    """Calls into the kernel libraries so far, over all loaded libraries."""
    return sum(lib.calls for lib in _loaded.values())


def loaded_libraries() -> Dict[str, str]:
    return {name: lib.path for name, lib in _loaded.items()}


def library(name: str) -> KernelLibrary:
    lib = _loaded.get(name)
    if lib is None:
        with _lock:
            lib = _loaded.get(name)
            if lib is None:
                lib = KernelLibrary(name)
                _loaded[name] = lib
    return lib
