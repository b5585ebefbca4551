"""Thin numpy-facing helpers over the device-resident C API: device arrays, packed-weight
handles and the fused ternary linear call.  Used by the runtime's callers that want to keep
activations on the GPU between calls, by the tests and by the benchmark."""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import numpy as np

from . import kernel as _k


class DeviceArray:
    """A typed, shaped view of GPU memory obtained from ``lspk_malloc``."""

    def __init__(self, shape, dtype):
        self.lib = _k.load_library(True)
        self.shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list)) else (shape,)))
        self.dtype = np.dtype(dtype)
        self.nbytes = int(np.prod(self.shape, dtype=np.int64)) * self.dtype.itemsize
        self.ptr = self.lib.lspk_malloc(self.nbytes)
        if not self.ptr:
            raise _k.KernelError(_k.last_error())

    @classmethod
    def from_numpy(cls, a: np.ndarray) -> "DeviceArray":
        a = np.ascontiguousarray(a)
        d = cls(a.shape, a.dtype)
        _k.check(d.lib.lspk_h2d(d.ptr, a.ctypes.data, d.nbytes))
        return d

    def copy_from(self, a: np.ndarray) -> None:
        a = np.ascontiguousarray(a, dtype=self.dtype)
        assert a.nbytes == self.nbytes
        _k.check(self.lib.lspk_h2d(self.ptr, a.ctypes.data, self.nbytes))

    def numpy(self) -> np.ndarray:
        out = np.empty(self.shape, dtype=self.dtype)
        _k.check(self.lib.lspk_d2h(out.ctypes.data, self.ptr, self.nbytes))
        return out

    def fill_bytes(self, value: int = 0) -> None:
        _k.check(self.lib.lspk_memset(self.ptr, value, self.nbytes))

    def free(self) -> None:
        if getattr(self, "ptr", None):
            self.lib.lspk_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class DeviceWeight:
    """A packed ternary matrix in the device layout (``lspk_upload_packed``)."""

    def __init__(self, packed: np.ndarray, scale: float, K: Optional[int] = None):
        self.lib = _k.load_library(True)
        packed = np.ascontiguousarray(packed, dtype=np.uint8)
        self.N, Kb = packed.shape
        self.K = int(K) if K is not None else Kb * 4
        self.scale = float(np.float32(scale))
        self.handle = self.lib.lspk_upload_packed(packed, self.N, self.K, self.scale)
        if not self.handle:
            raise _k.KernelError(_k.last_error())
        self.owned = True

    @property
    def device_bytes(self) -> int:
        b = ctypes.c_size_t(0)
        _k.check(self.lib.lspk_weight_shape(self.handle, None, None, None, ctypes.byref(b)))
        return int(b.value)

    def download(self) -> np.ndarray:
        out = np.empty((self.N, self.K // 4), dtype=np.uint8)
        _k.check(self.lib.lspk_download_packed(self.handle, out))
        return out

    def free(self) -> None:
        if getattr(self, "handle", None) and self.owned:
            self.lib.lspk_weight_free(self.handle)
        self.handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def linear(weights: Sequence, outs: Sequence[Optional[DeviceArray]], M: int, *, x_f32: Optional[DeviceArray] = None,
           x_i8: Optional[DeviceArray] = None, x_scales: Optional[DeviceArray] = None,
           gamma: Optional[DeviceArray] = None, gate_f32: Optional[DeviceArray] = None, eps: float = 1e-5,
           epilogue: int = _k.EPI_STORE,
           acc_outs: Sequence[Optional[DeviceArray]] = (), xq_out: Optional[DeviceArray] = None,
           xscale_out: Optional[DeviceArray] = None) -> None:
    """Call ``lspk_linear``.  The prologue follows from the inputs given: int8 + scales ->
    LSPK_PRO_INT8; fp32 -> fused quantiser; fp32 + gamma -> fused RMSNorm + quantiser."""
    lib = _k.load_library(True)
    a = _k.LinearArgs()
    for i, w in enumerate(weights):
        a.w[i] = w.handle if hasattr(w, "handle") else w
    for i, o in enumerate(outs):
        a.out[i] = o.ptr if o is not None else None
    for i, o in enumerate(acc_outs):
        a.acc_out[i] = o.ptr if o is not None else None
    a.n_mats = len(weights)
    a.M = int(M)
    a.epilogue = int(epilogue)
    a.eps = float(eps)
    if x_i8 is not None:
        a.prologue = _k.PRO_INT8
        a.x_i8 = x_i8.ptr
        a.x_scales = x_scales.ptr
    else:
        a.x_f32 = x_f32.ptr
        if gate_f32 is not None:
            a.gate_f32 = gate_f32.ptr
        if gamma is not None:
            a.prologue = _k.PRO_GATED_RMSNORM_QUANT if gate_f32 is not None else _k.PRO_RMSNORM_QUANT
            a.gamma = gamma.ptr
            a.gamma_is_bf16 = int(gamma.dtype == np.uint16)
        else:
            a.prologue = _k.PRO_QUANT
    a.xq_out = xq_out.ptr if xq_out is not None else None
    a.xscale_out = xscale_out.ptr if xscale_out is not None else None
    _k.check(lib.lspk_linear(ctypes.byref(a)))


def sync() -> None:
    _k.check(_k.load_library(True).lspk_sync())


class Timer:
    """CUDA-event timing on the library's stream."""

    def __enter__(self):
        self.lib = _k.load_library(True)
        _k.check(self.lib.lspk_timer_start())
        return self

    def __exit__(self, *exc):
        ms = ctypes.c_float(0.0)
        _k.check(self.lib.lspk_timer_stop(ctypes.byref(ms)))
        self.ms = float(ms.value)
        return False
