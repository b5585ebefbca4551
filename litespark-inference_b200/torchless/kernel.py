"""ctypes boundary to the sm_100a library -- the drop-in for the reference's
``litespark_inference/torchless/kernel.py``.

The arch-neutral wrapper names, argument order, dtypes and return values below are the ones
``runtime.py`` of the reference imports (``kernel.py:328-741`` there); the C symbols behind
them carry the tag ``sm100`` instead of ``avx512`` / ``avx2`` / ``neon``.  Arrays are host
numpy arrays, exactly as with the reference: each call stages them through the GPU.  For
performance use the device-resident API (``runtime.py`` of this package), which keeps weights,
activations and the KV cache on the GPU.

There is no CPU fallback.  Importing works anywhere; the first kernel call raises
``KernelUnavailable`` if the shared library is missing or no sm_100 GPU is present.
"""
from __future__ import annotations

import ctypes
from pathlib import Path
from typing import Optional

import numpy as np
from numpy import ctypeslib as _npct

_PKG = Path(__file__).resolve().parent.parent
_LIB_PATH = _PKG / "_lspk_sm100.so"
_ARCH_TAG = "sm100"
_lib: Optional[ctypes.CDLL] = None


class KernelUnavailable(RuntimeError):
    pass


class KernelError(RuntimeError):
    pass


_F32 = _npct.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_I8 = _npct.ndpointer(dtype=np.int8, flags="C_CONTIGUOUS")
_U8 = _npct.ndpointer(dtype=np.uint8, flags="C_CONTIGUOUS")
_U16 = _npct.ndpointer(dtype=np.uint16, flags="C_CONTIGUOUS")
_ci, _cf, _vp, _sz = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t


class LinearArgs(ctypes.Structure):
    """Mirror of ``lspk_linear_args`` (include/lspk_sm100.h)."""
    _fields_ = [
        ("w", _vp * 3), ("out", _vp * 3), ("n_mats", _ci), ("M", _ci),
        ("prologue", _ci), ("epilogue", _ci),
        ("x_f32", _vp), ("x_i8", _vp), ("x_scales", _vp),
        ("gamma", _vp), ("gamma_is_bf16", _ci), ("eps", _cf),
        ("acc_out", _vp * 3), ("xq_out", _vp), ("xscale_out", _vp), ("gate_f32", _vp),
    ]


PRO_INT8, PRO_QUANT, PRO_RMSNORM_QUANT, PRO_GATED_RMSNORM_QUANT = 0, 1, 2, 3
EPI_STORE, EPI_ADD, EPI_RELU2_MUL, EPI_SILU_MUL = 0, 1, 2, 3

# name -> (argtypes, restype) of every symbol declared in include/lspk_sm100.h
_SIGNATURES = {
    "lspk_init": ([_ci], _ci),
    "lspk_device_count": ([], _ci),
    "lspk_mem_info": ([ctypes.POINTER(_sz), ctypes.POINTER(_sz)], _ci),
    "lspk_sm_count": ([], _ci),
    "lspk_last_error": ([], ctypes.c_char_p),
    "lspk_error_count": ([], _ci),
    "lspk_clear_error": ([], None),
    "lspk_set_pdl": ([_ci], _ci),
    "lspk_sync": ([], _ci),
    "lspk_malloc": ([_sz], _vp),
    "lspk_free": ([_vp], _ci),
    "lspk_host_alloc": ([_sz], _vp),
    "lspk_host_free": ([_vp], _ci),
    "lspk_h2d": ([_vp, _vp, _sz], _ci),
    "lspk_d2h": ([_vp, _vp, _sz], _ci),
    "lspk_h2d_async": ([_vp, _vp, _sz], _ci),
    "lspk_d2h_async": ([_vp, _vp, _sz], _ci),
    "lspk_memset": ([_vp, _ci, _sz], _ci),
    "lspk_flush_l2": ([], _ci),
    "lspk_trace_begin": ([_ci], _ci),
    "lspk_trace_read": ([_vp, _ci, ctypes.POINTER(_ci)], _ci),
    "lspk_timer_start": ([], _ci),
    "lspk_timer_stop": ([ctypes.POINTER(_cf)], _ci),
    "lspk_upload_packed": ([_U8, _ci, _ci, _cf], _vp),
    "lspk_upload_bf16_ternary": ([_vp, _ci, _ci, ctypes.c_double], _vp),
    "lspk_download_packed": ([_vp, _U8], _ci),
    "lspk_weight_free": ([_vp], _ci),
    "lspk_weight_shape": ([_vp, ctypes.POINTER(_ci), ctypes.POINTER(_ci), ctypes.POINTER(_cf),
                           ctypes.POINTER(_sz)], _ci),
    "lspk_linear": ([ctypes.POINTER(LinearArgs)], _ci),
    "lspk_linear_force_path": ([_ci], _ci),
    "lspk_linear_batch": ([ctypes.POINTER(LinearArgs), _ci], _ci),
    "lspk_tc_check_error": ([], _ci),
    "lspk_quantize_rows": ([_vp, _vp, _vp, _ci, _ci], _ci),
    "lspk_rmsnorm_rows": ([_vp, _vp, _ci, _vp, _ci, _ci, _cf], _ci),
    "lspk_rmsnorm_quantize_rows": ([_vp, _vp, _ci, _vp, _vp, _ci, _ci, _cf], _ci),
    "lspk_relu2_mul_rows": ([_vp, _vp, _vp, _ci, _ci], _ci),
    "lspk_add_rows": ([_vp, _vp, _sz], _ci),
    "lspk_lm_head": ([_ci, _vp, _vp, _vp, _vp, _ci, _ci, _ci], _ci),
    "matmul_lut_sm100_m1": ([_I8, _U8, _cf, _cf, _F32, _ci, _ci], None),
    "matmul_lut_sm100_mT": ([_I8, _F32, _U8, _cf, _F32, _ci, _ci, _ci], None),
    "matmul_lut_sm100_prefill": ([_I8, _U8, _cf, _F32, _F32, _ci, _ci, _ci], None),
    "quantize_activation_sm100": ([_F32, _I8, _ci], _cf),
    "quantize_activation_batched_sm100": ([_F32, _I8, _F32, _ci, _ci], None),
    "rmsnorm_bf16gamma_fp32_sm100": ([_F32, _U16, _F32, _ci, _cf], None),
    "rmsnorm_fp32gamma_fp32_sm100": ([_F32, _F32, _F32, _ci, _cf], None),
    "rmsnorm_bf16gamma_fp32_batched_sm100": ([_F32, _U16, _F32, _ci, _ci, _cf], None),
    "rmsnorm_fp32gamma_fp32_batched_sm100": ([_F32, _F32, _F32, _ci, _ci, _cf], None),
    "rmsnorm_quantize_bf16gamma_sm100": ([_F32, _U16, _I8, _F32, _ci, _cf], _cf),
    "rmsnorm_quantize_bf16gamma_batched_sm100": ([_F32, _U16, _I8, _F32, _F32, _ci, _ci, _cf], None),
    "relu2_mul_fp32_sm100": ([_F32, _F32, _F32, _ci], None),
    "relu2_mul_fp32_batched_sm100": ([_F32, _F32, _F32, _ci, _ci], None),
    "add_inplace_fp32_sm100": ([_F32, _F32, _ci], None),
    "lm_head_bf16_fp32_sm100": ([_U16, _F32, _F32, _ci, _ci], None),
    "lm_head_int8_fp32_sm100": ([_I8, _F32, _F32, _F32, _ci, _ci], None),
    "lm_head_int4_fp32_sm100": ([_U8, _F32, _F32, _F32, _ci, _ci], None),
    "matmul_lut_sm100_m1_noalloc": ([_I8, _U8, _cf, _cf, _F32, _ci, _ci], _ci),
    "matmul_lut_sm100_has_omp": ([], _ci),
    "matmul_lut_sm100_max_threads": ([], _ci),
    "lspk_register_packed": ([_U8, _ci, _ci], _ci),
    "lspk_register_embedding": ([_ci, _vp, _vp, _ci, _ci], _ci),
    "lspk_unregister": ([_vp], _ci),
    "lspk_unregister_all": ([], _ci),
}

# reference-neutral alias -> tagged C symbol (the aliasing the reference does in kernel.py:227-322)
_ALIASES = {
    "matmul_lut_m1": "matmul_lut_{T}_m1",
    "matmul_lut_mT": "matmul_lut_{T}_mT",
    "matmul_lut_prefill": "matmul_lut_{T}_prefill",
    "quantize_activation": "quantize_activation_{T}",
    "quantize_activation_batched": "quantize_activation_batched_{T}",
    "rmsnorm_bf16gamma_fp32": "rmsnorm_bf16gamma_fp32_{T}",
    "rmsnorm_fp32gamma_fp32": "rmsnorm_fp32gamma_fp32_{T}",
    "rmsnorm_bf16gamma_fp32_batched": "rmsnorm_bf16gamma_fp32_batched_{T}",
    "rmsnorm_fp32gamma_fp32_batched": "rmsnorm_fp32gamma_fp32_batched_{T}",
    "rmsnorm_quantize_bf16gamma": "rmsnorm_quantize_bf16gamma_{T}",
    "rmsnorm_quantize_bf16gamma_batched": "rmsnorm_quantize_bf16gamma_batched_{T}",
    "relu2_mul_fp32": "relu2_mul_fp32_{T}",
    "relu2_mul_fp32_batched": "relu2_mul_fp32_batched_{T}",
    "add_inplace_fp32": "add_inplace_fp32_{T}",
    "lm_head_bf16_fp32": "lm_head_bf16_fp32_{T}",
    "lm_head_int8_fp32": "lm_head_int8_fp32_{T}",
    "lm_head_int4_fp32": "lm_head_int4_fp32_{T}",
    "has_omp_probe": "matmul_lut_{T}_has_omp",
    "max_threads_probe": "matmul_lut_{T}_max_threads",
}


def library_path() -> Path:
    return _LIB_PATH


def load_library(require_device: bool = True) -> ctypes.CDLL:
    """dlopen the shared library and bind every declared symbol.  With require_device the GPU
    is initialised too (raises KernelUnavailable when there is none)."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise KernelUnavailable(
                f"{_LIB_PATH} is missing: build it with `python {_PKG.name}/build.py` "
                "(there is no CPU fallback)")
        lib = ctypes.CDLL(str(_LIB_PATH))
        for name, (argtypes, restype) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = restype
        for neutral, tagged in _ALIASES.items():
            setattr(lib, neutral, getattr(lib, tagged.format(T=_ARCH_TAG)))
        try:
            from . import _bench_abi, _runtime_abi
            _runtime_abi.bind(lib)
            _bench_abi.bind(lib)
        except ImportError:
            pass
        _lib = lib
    if require_device and not getattr(_lib, "_device_ready", False):
        if _lib.lspk_init(int(__import__("os").environ.get("LITESPARK_DEVICE", "0"))) != 0:
            raise KernelUnavailable(_lib.lspk_last_error().decode() or "no usable sm_100 GPU")
        _lib._device_ready = True
    return _lib


def _load() -> ctypes.CDLL:
    return load_library(True)


def last_error() -> str:
    return load_library(False).lspk_last_error().decode()


class _ErrorGuard:
    """The drop-in symbols return void like the reference's; surface recorded failures as
    exceptions on the Python side."""

    def __enter__(self):
        self.lib = _load()
        self.before = self.lib.lspk_error_count()
        return self.lib

    def __exit__(self, et, ev, tb):
        if et is None and self.lib.lspk_error_count() != self.before:
            raise KernelError(self.lib.lspk_last_error().decode())
        return False


def check(rc: int) -> None:
    if rc != 0:
        raise KernelError(f"[{rc}] {last_error()}")


# ---------------------------------------------------------------------------------------------
# probes (reference kernel.py:328-338, 462-484, 519-538)
# ---------------------------------------------------------------------------------------------
def has_omp() -> bool:
    return bool(_load().has_omp_probe())


def max_threads() -> int:
    """The reference reports OpenMP threads; here: the number of SMs of the GPU."""
    return int(_load().max_threads_probe())


def has_accelerate() -> bool:
    return False


def has_unpacked_matmul() -> bool:
    """One byte per weight would quadruple the HBM traffic; not offered."""
    return False


def has_batched_matmul() -> bool:
    return True


def has_batched_helpers() -> bool:
    return True


def has_fused_rmsnorm_quantize() -> bool:
    return True


def has_amx() -> bool:
    return False


def ensure_built() -> Path:
    load_library(False)
    return _LIB_PATH


# ---------------------------------------------------------------------------------------------
# wrappers with the reference's names and signatures (host numpy arrays)
# ---------------------------------------------------------------------------------------------
def lm_head_int4(emb_packed, emb_scale, x_fp32, out_fp32, H: int):
    with _ErrorGuard() as lib:
        lib.lm_head_int4_fp32(emb_packed, emb_scale, x_fp32, out_fp32, emb_packed.shape[0], H)
    return out_fp32


def lm_head_int8(emb_int8, emb_scale, x_fp32, out_fp32):
    V, H = emb_int8.shape
    with _ErrorGuard() as lib:
        lib.lm_head_int8_fp32(emb_int8, emb_scale, x_fp32, out_fp32, V, H)
    return out_fp32


def lm_head_bf16(emb_u16, x_fp32, out_fp32):
    V, H = emb_u16.shape
    with _ErrorGuard() as lib:
        lib.lm_head_bf16_fp32(emb_u16, x_fp32, out_fp32, V, H)
    return out_fp32


def rmsnorm_into(x_fp32, gamma, out_fp32, eps: float = 1e-5):
    K = x_fp32.shape[0]
    with _ErrorGuard() as lib:
        if gamma.dtype == np.uint16:
            lib.rmsnorm_bf16gamma_fp32(x_fp32, gamma, out_fp32, K, eps)
        elif gamma.dtype == np.float32:
            lib.rmsnorm_fp32gamma_fp32(x_fp32, gamma, out_fp32, K, eps)
        else:
            raise TypeError(f"gamma dtype must be uint16 or float32, got {gamma.dtype}")
    return out_fp32


def rmsnorm_into_batched(x_fp32, gamma, out_fp32, eps: float = 1e-5):
    T, K = x_fp32.shape
    with _ErrorGuard() as lib:
        if gamma.dtype == np.uint16:
            lib.rmsnorm_bf16gamma_fp32_batched(x_fp32, gamma, out_fp32, T, K, eps)
        elif gamma.dtype == np.float32:
            lib.rmsnorm_fp32gamma_fp32_batched(x_fp32, gamma, out_fp32, T, K, eps)
        else:
            raise TypeError(f"gamma dtype must be uint16 or float32, got {gamma.dtype}")
    return out_fp32


def relu2_mul_into(gate_fp32, up_fp32, out_fp32):
    with _ErrorGuard() as lib:
        lib.relu2_mul_fp32(gate_fp32, up_fp32, out_fp32, gate_fp32.shape[0])
    return out_fp32


def relu2_mul_into_batched(gate_fp32, up_fp32, out_fp32):
    T, K = gate_fp32.shape
    with _ErrorGuard() as lib:
        lib.relu2_mul_fp32_batched(gate_fp32, up_fp32, out_fp32, T, K)
    return out_fp32


def add_inplace(a_fp32, b_fp32):
    with _ErrorGuard() as lib:
        lib.add_inplace_fp32(a_fp32, b_fp32, a_fp32.shape[0])
    return a_fp32


def quantize_activation(x_fp32, out_int8) -> float:
    with _ErrorGuard() as lib:
        return float(lib.quantize_activation(x_fp32, out_int8, x_fp32.shape[0]))


def quantize_activation_batched(x_fp32, out_int8, out_scales):
    T, K = x_fp32.shape
    with _ErrorGuard() as lib:
        lib.quantize_activation_batched(x_fp32, out_int8, out_scales, T, K)
    return out_scales


def rmsnorm_quantize_into(x_fp32, gamma, x_int8_out, tmp_fp32, eps: float = 1e-5) -> float:
    with _ErrorGuard() as lib:
        return float(lib.rmsnorm_quantize_bf16gamma(x_fp32, gamma, x_int8_out, tmp_fp32, x_fp32.shape[0], eps))


def rmsnorm_quantize_batched(x_fp32, gamma, x_int8_out, scales_out, tmp_fp32, eps: float = 1e-5):
    T, K = x_fp32.shape
    with _ErrorGuard() as lib:
        lib.rmsnorm_quantize_bf16gamma_batched(x_fp32, gamma, x_int8_out, scales_out, tmp_fp32, T, K, eps)
    return scales_out


def matmul_packed_m1(x_int8, packed_w, w_scale: float, x_scale: float, out=None):
    """Ternary GEMV, M = 1 (reference kernel.py:423-448)."""
    N, Kb = packed_w.shape
    if out is None:
        out = np.empty(N, dtype=np.float32)
    with _ErrorGuard() as lib:
        lib.matmul_lut_m1(x_int8, packed_w, w_scale, x_scale, out, N, Kb * 4)
    return out


def matmul_packed_m1_noalloc(x_int8, packed_w, w_scale: float, x_scale: float, out=None):
    """``matmul_packed_m1`` for hosts that may not allocate GPU memory when they call (all memory
    already owned by a serving framework's pool, or an allocation-free real-time loop).  The device
    scratch is a fixed 12 MiB array inside the library, so the matrix must fit it (6912 x 2560
    does); a larger one raises KernelError.  Make the first call outside any CUDA stream capture."""
    N, Kb = packed_w.shape
    if out is None:
        out = np.empty(N, dtype=np.float32)
    check(_load().matmul_lut_sm100_m1_noalloc(x_int8, packed_w, w_scale, x_scale, out, N, Kb * 4))
    return out


def matmul_packed_mT(x_int8, x_scales, packed_w, w_scale: float, out=None):
    """Batched ternary matmul, any T >= 1 (reference kernel.py:625-651)."""
    T, K = x_int8.shape
    N, Kb = packed_w.shape
    assert Kb * 4 == K, f"K mismatch: {K} vs Kb*4={Kb * 4}"
    if out is None:
        out = np.empty((T, N), dtype=np.float32)
    with _ErrorGuard() as lib:
        lib.matmul_lut_mT(x_int8, x_scales, packed_w, w_scale, out, T, N, K)
    return out


def matmul_packed_prefill(x_int8, packed_w, w_scale: float, x_scale, out=None):
    """Same product with the reference's ARM argument order (kernel.py:678-734)."""
    x_int8 = np.ascontiguousarray(x_int8)
    packed_w = np.ascontiguousarray(packed_w)
    M, K = x_int8.shape
    N, Kb = packed_w.shape
    if Kb * 4 != K:
        raise ValueError(f"x K={K} != K={Kb * 4} implied by packed_w")
    x_scale = np.ascontiguousarray(x_scale, dtype=np.float32)
    if x_scale.shape != (M,):
        raise ValueError(f"x_scale must be float32 [M={M}], got {x_scale.shape}")
    if out is None:
        out = np.empty((M, N), dtype=np.float32)
    elif out.shape != (M, N) or out.dtype != np.float32:
        raise ValueError("out must be float32 [M, N]")
    with _ErrorGuard() as lib:
        lib.matmul_lut_prefill(x_int8, packed_w, w_scale, x_scale, out, M, N, K)
    return out


def matmul_unpacked_m1(*_a, **_k):
    raise RuntimeError("pre-unpacked weights are not supported on the GPU path (has_unpacked_matmul() is False)")


def matmul_accelerate_f32_m1(*_a, **_k):
    raise RuntimeError("mode='accelerate' requires Apple Accelerate")


def matmul_amx_mT(*_a, **_k):
    raise RuntimeError("AMX is a CPU feature (has_amx() is False); use matmul_packed_mT")


matmul_amx_mT_padded = matmul_amx_mT


# ---------------------------------------------------------------------------------------------
# weight residency for the drop-ins
# ---------------------------------------------------------------------------------------------
def register_packed(packed_w: np.ndarray) -> None:
    """Keep a device copy of this packed matrix; later drop-in calls given the same array skip
    the upload.  The array must stay alive and unmodified."""
    N, Kb = packed_w.shape
    check(_load().lspk_register_packed(packed_w, N, Kb * 4))


def register_embedding(emb: np.ndarray, emb_scale: Optional[np.ndarray] = None, H: Optional[int] = None) -> None:
    kind = {np.dtype(np.uint16): 0, np.dtype(np.int8): 1, np.dtype(np.uint8): 2}[emb.dtype]
    V = emb.shape[0]
    H = H or (emb.shape[1] * (2 if kind == 2 else 1))
    sp = emb_scale.ctypes.data if emb_scale is not None else None
    check(_load().lspk_register_embedding(kind, emb.ctypes.data, sp, V, H))


def unregister_all() -> None:
    check(_load().lspk_unregister_all())
