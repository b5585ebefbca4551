"""ctypes signatures of include/lspk_runtime.h."""
import ctypes

_ci, _cf, _vp, _sz = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t


class ModelConfig(ctypes.Structure):
    """Mirror of ``lspk_model_config``."""
    _fields_ = [("hidden_size", _ci), ("num_layers", _ci), ("num_heads", _ci), ("num_kv_heads", _ci),
                ("intermediate_size", _ci), ("vocab_size", _ci), ("rms_norm_eps", _cf), ("arch", _ci)]


SIGNATURES = {
    "lspk_model_create": ([ctypes.POINTER(ModelConfig)], _vp),
    "lspk_model_set_projection": ([_vp, _ci, _ci, _vp, _ci, _ci, _cf], _ci),
    "lspk_model_set_projection_bf16": ([_vp, _ci, _ci, _vp, _ci, _ci, ctypes.c_double], _ci),
    "lspk_model_set_norm": ([_vp, _ci, _ci, _vp, _ci, _ci], _ci),
    "lspk_model_set_embedding": ([_vp, _ci, _vp, _vp], _ci),
    "lspk_model_set_lm_head": ([_vp, _ci, _vp, _vp], _ci),
    "lspk_model_finalize": ([_vp], _ci),
    "lspk_model_device_bytes": ([_vp], _sz),
    "lspk_model_projection": ([_vp, _ci, _ci], _vp),
    "lspk_model_free": ([_vp], _ci),
    "lspk_state_create": ([_vp, _ci, _ci, _ci, _vp, _vp], _vp),
    "lspk_state_free": ([_vp], _ci),
    "lspk_state_get_pos": ([_vp, _ci], _ci),
    "lspk_state_set_pos": ([_vp, _ci, _ci], _ci),
    "lspk_state_device_bytes": ([_vp], _sz),
    "lspk_state_read_kv": ([_vp, _ci, _ci, _ci, _vp, _vp], _ci),
    "lspk_forward_step": ([_vp, _vp, _vp, _vp], _ci),
    "lspk_forward_prefill": ([_vp, _ci, _vp, _ci, _vp, _vp, _vp], _ci),
    "lspk_decode_greedy": ([_vp, _vp, _ci, _vp], _ci),
    "lspk_state_step_kernel_count": ([_vp], _ci),
    "lspk_debug_expire_wait": ([_ci], _ci),
}


def bind(lib) -> None:
    for name, (argtypes, restype) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = restype
