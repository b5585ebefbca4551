"""ctypes signatures of include/lspk_bench.h (measurement-only entry points, used by bench.py)."""
import ctypes

_ci, _cf, _vp, _sz = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t
_pf, _pd, _pi = ctypes.POINTER(_cf), ctypes.POINTER(ctypes.c_double), ctypes.POINTER(_ci)

SIGNATURES = {
    "lspk_bench_handoff": ([_ci, _ci, _ci, _pf, _pd], _ci),
    "lspk_bench_cluster": ([_ci, _ci, _ci, _ci, _ci, _ci, _pf], _ci),
    "lspk_bench_linears": ([_vp, _ci, ctypes.POINTER(_cf), ctypes.POINTER(_ci), ctypes.POINTER(ctypes.c_double)], _ci),
    "lspk_bench_linear_copies": ([_vp, _ci, _vp, _vp, _ci, _ci, ctypes.POINTER(_cf)], _ci),
    "lspk_bench_launch_floor": ([_ci, _ci, _ci, ctypes.POINTER(_cf)], _ci),
    "lspk_bench_linear_copies_independent": ([_vp, _vp, _ci, _vp, _vp, _ci, _ci, _ci, _ci, ctypes.POINTER(_cf)], _ci),
    "lspk_bench_lm_head": ([_vp, _ci, ctypes.POINTER(_cf), ctypes.POINTER(ctypes.c_double)], _ci),
    "lspk_tp_bench_mlp": ([_vp, _vp, _vp, _ci, _vp, _vp, _vp, _cf, _vp, _vp, _vp, _vp, _ci, ctypes.POINTER(_cf)], _ci),
}


def bind(lib) -> None:
    for name, (argtypes, restype) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = restype
