"""ctypes signatures of include/lspk_bench.h (measurement-only entry points, used by bench.py)."""
import ctypes

_ci, _cf, _vp = ctypes.c_int, ctypes.c_float, ctypes.c_void_p
_pf, _pd, _pi = ctypes.POINTER(_cf), ctypes.POINTER(ctypes.c_double), ctypes.POINTER(_ci)

SIGNATURES = {
    "lspk_bench_handoff": ([_ci, _ci, _ci, _pf, _pd], _ci),
}


def bind(lib) -> None:
    for name, (argtypes, restype) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = restype
