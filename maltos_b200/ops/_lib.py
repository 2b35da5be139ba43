"""ctypes binding to ``libmaltos_b200.so`` (the sm_100a kernel library).

The library is built in-tree by :mod:`maltos_b200.build`. On a machine with a CUDA device the ops in
this package refuse to run without it (no silent eager fallback); on CPU-only machines the library is
never loaded and the ops use their PyTorch fp32 restatements, which are also the oracles of the GPU tests.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent.parent / "libmaltos_b200.so"
_lib = None
_lock = threading.Lock()

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float
c_double = ctypes.c_double


class KernelLibraryError(RuntimeError):
    """Raised when the kernel library is missing, fails to load, or a launcher reports an error."""


class DeviceStatusError(RuntimeError):
    """Raised when a kernel left an error code in the per-device status word (bounded wait ran out...)."""


class CommTimeoutError(DeviceStatusError):
    """A bounded wait on a flag that another rank writes ran out: the peer never delivered. ``peer`` is the rank (within
    the op's process group) whose flag was missing; the kernel returned cleanly and the context stays usable."""

    def __init__(self, message: str, *, peer: int, block: int) -> None:
        super().__init__(message)
        self.peer, self.block = peer, block


# ------------------------------------------------------------------------------------------------ NVTX ranges
def nvtx_enabled() -> bool:
    """``MALTOS_B200_NVTX=1``: every launcher call of the library runs inside an NVTX range named after the C entry point
    (``mb_gemm_bf16``, ``mb_flash_attn_bwd``, ...), so a timeline tool shows which op issued which kernels."""
    return os.environ.get("MALTOS_B200_NVTX", "0") == "1"


def _range_push(name: str) -> None:
    torch.cuda.nvtx.range_push(name)


def _range_pop() -> None:
    torch.cuda.nvtx.range_pop()


#: entry points that launch nothing (queries, setters): no range around them
_NO_RANGE = ("mb_last_error", "mb_launch_count", "mb_set_", "mb_status_", "mb_flash_attn_bwd_scratch_words", "mb_symm_", "mb_gemm_set_")


class _RangedFunction:
    """A C entry point whose calls are bracketed by an NVTX range; ``restype`` / ``argtypes`` go to the real function."""

    __slots__ = ("_fn", "_name")

    def __init__(self, fn, name: str) -> None:
        object.__setattr__(self, "_fn", fn)
        object.__setattr__(self, "_name", name)

    def __call__(self, *args):
        _range_push(self._name)
        try:
            return self._fn(*args)
        finally:
            _range_pop()

    def __getattr__(self, item):
        return getattr(self._fn, item)

    def __setattr__(self, item, value) -> None:
        setattr(self._fn, item, value)


class _RangedLibrary:
    """The kernel library with NVTX ranges around its launchers (see :func:`nvtx_enabled`)."""

    def __init__(self, handle) -> None:
        self.__dict__["_handle"] = handle
        self.__dict__["_cache"] = {}

    def __getattr__(self, name: str):
        fn = getattr(self._handle, name)
        if not name.startswith("mb_") or name.startswith(_NO_RANGE):
            return fn
        wrapped = self._cache.get(name)
        if wrapped is None:
            wrapped = self._cache[name] = _RangedFunction(fn, name)
        return wrapped


def library_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    return _LIB_PATH.exists()


def lib() -> ctypes.CDLL:
    """Load (once) and return the kernel library. Raises :class:`KernelLibraryError` if it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not _LIB_PATH.exists():
            if os.environ.get("MALTOS_B200_AUTOBUILD", "1") == "1":
                try:
                    from maltos_b200 import build as _build

                    _build.build()
                except Exception as exc:  # pragma: no cover - depends on toolchain
                    raise KernelLibraryError(
                        f"{_LIB_PATH} is missing and building it failed: {exc}. "
                        "Run `python -m maltos_b200.build` on a machine with nvcc."
                    ) from exc
            else:
                raise KernelLibraryError(f"{_LIB_PATH} is missing; run `python -m maltos_b200.build`")
        try:
            handle = ctypes.CDLL(str(_LIB_PATH))
        except OSError as exc:
            raise KernelLibraryError(f"cannot load {_LIB_PATH}: {exc}") from exc
        handle.mb_last_error.restype = ctypes.c_char_p
        handle.mb_launch_count.restype = ctypes.c_ulonglong
        _lib = _RangedLibrary(handle) if nvtx_enabled() else handle
    return _lib


def use_kernels(*tensors: torch.Tensor) -> bool:
    """True when the tensors live on a CUDA device (so the sm_100a kernels are the path to run)."""
    return any(t is not None and t.is_cuda for t in tensors)


def stream_ptr() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: torch.Tensor | None) -> c_void_p:
    if t is None:
        return c_void_p(0)
    return c_void_p(t.data_ptr())


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().mb_last_error().decode(errors="replace")
        raise KernelLibraryError(f"{what} failed (code {rc}): {msg}")


def set_wait_timeout_ms(ms: int) -> None:
    """Limit of every bounded device-side wait on the current device (0 restores the default of 4 s)."""
    check(lib().mb_set_wait_timeout_ms(c_int(int(ms))), "mb_set_wait_timeout_ms")


def launch_count() -> int:
    """Number of kernels launched by this library in this process so far (0 if it was never loaded)."""
    if _lib is None:
        return 0
    return int(_lib.mb_launch_count())


def fetch_status(raise_on_error: bool = True) -> tuple[int, int, int, int]:
    """Synchronise the current stream, read and clear the device status word.

    Kernels never trap or spin forever: a wait that runs out of time sets a bit here and the kernel
    returns. ``(code, block, detail, _)``; ``code`` 0 means no error since the last fetch.
    """
    out = (ctypes.c_int * 4)()
    check(lib().mb_status_fetch_and_clear(out, stream_ptr()), "mb_status_fetch_and_clear")
    vals = tuple(int(v) for v in out)
    if raise_on_error and vals[0] != 0:
        names = []
        if vals[0] & 1:
            names.append("mbarrier wait timed out")
        if vals[0] & 2:
            names.append("peer flag wait timed out")
        if vals[0] & 4:
            names.append("index out of bounds")
        msg = f"kernel status {vals[0]} ({', '.join(names)}); block {vals[1]}, detail {vals[2]}"
        if vals[0] & 2:
            raise CommTimeoutError(msg, peer=vals[2], block=vals[1])
        raise DeviceStatusError(msg)
    return vals  # type: ignore[return-value]
