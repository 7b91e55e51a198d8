"""Device/context handle — the counterpart of hyperscalees-core
(hyperscalees-core/src/lib.rs:6-23: `type B`, `default_device()`, `is_gpu()`).

The backend is fixed: CUDA on a B200.  `default_device()` returns the current
CUDA device and fails when none is present; `is_gpu()` is therefore always
true once a device exists.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict

import torch

from . import _lib


def is_gpu() -> bool:
    """hyperscalees-core/src/lib.rs:19-23.  No CPU backend is compiled in."""
    return True


def default_device() -> torch.device:
    """hyperscalees-core/src/lib.rs:12-17."""
    if not torch.cuda.is_available():
        raise RuntimeError("hyperscalees_b200 needs a CUDA device (no CPU backend exists)")
    return torch.device("cuda", torch.cuda.current_device())


class Context:
    """Owns an `hses_ctx` for one device (jump tables + libm calibration)."""

    def __init__(self, device: int):
        self._lib = _lib.load()
        handle = C.c_void_p()
        _lib.check(self._lib.hses_ctx_create(int(device), C.byref(handle)))
        self.handle = handle
        self.device = int(device)

    def calibration_info(self):
        a, b = C.c_uint64(), C.c_uint64()
        _lib.check(self._lib.hses_ctx_calibration_info(self.handle, C.byref(a), C.byref(b)))
        return int(a.value), int(b.value)

    def device_status(self) -> int:
        """Synchronises and returns the code a kernel left when a bounded wait ran out (0 = none)."""
        st = C.c_int()
        _lib.check(self._lib.hses_ctx_device_status(self.handle, C.byref(st)))
        return int(st.value)

    def profile_enable(self, timing: bool = True) -> None:
        """Clear the launch counters; with timing, bracket every launch with CUDA events."""
        _lib.check(self._lib.hses_profile_enable(self.handle, int(timing)))

    def profile_read(self):
        """{kernel name: (launches, total device ms)} since the last profile_enable."""
        out = {}
        for i in range(int(self._lib.hses_profile_count(self.handle))):
            name, n, ms = C.c_char_p(), C.c_int64(), C.c_double()
            _lib.check(self._lib.hses_profile_read(self.handle, i, C.byref(name), C.byref(n), C.byref(ms)))
            out[name.value.decode()] = (int(n.value), float(ms.value))
        return out

    def close(self):
        if self.handle:
            self._lib.hses_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_contexts: Dict[int, Context] = {}


def get_context(device=None) -> Context:
    """Process-wide context per CUDA device, created on first use."""
    if device is None:
        device = default_device()
    idx = device.index if isinstance(device, torch.device) else int(device)
    if idx is None:
        idx = torch.cuda.current_device()
    ctx = _contexts.get(idx)
    if ctx is None:
        with torch.cuda.device(idx):
            ctx = Context(idx)
        _contexts[idx] = ctx
    return ctx


def current_stream(device=None) -> int:
    """Raw cudaStream_t of torch's current stream (0 means the legacy default stream)."""
    return int(torch.cuda.current_stream(device).cuda_stream)
