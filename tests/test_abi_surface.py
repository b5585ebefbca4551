"""CPU-only checks of the boundary: the shared library loads without a GPU, exports every symbol
the headers declare, the ctypes layer binds every one of them, and the Python layer exposes the
wrapper names the reference's runtime imports."""
import ctypes
import importlib
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
K = importlib.import_module("litespark_inference_b200.torchless.kernel")


def _declared_symbols():
    names = set()
    for h in (ROOT / "include").glob("*.h"):
        text = re.sub(r"/\*.*?\*/", "", h.read_text(), flags=re.S)
        for m in re.finditer(r"^[A-Za-z_][\w\s\*]*?\b(\w+)\s*\([^;{]*\)\s*;", text, flags=re.M):
            names.add(m.group(1))
    return names


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(str(K.library_path()))
    declared = _declared_symbols()
    assert len(declared) > 60
    missing = [n for n in sorted(declared) if not hasattr(lib, n)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"


def test_ctypes_layer_binds_every_declared_symbol():
    lib = K.load_library(require_device=False)
    rt_abi = importlib.import_module("litespark_inference_b200.torchless._runtime_abi")
    hyb = importlib.import_module("litespark_inference_b200.torchless.hybrid")
    tpm = importlib.import_module("litespark_inference_b200.torchless.tp")
    bench_abi = importlib.import_module("litespark_inference_b200.torchless._bench_abi")
    bound = set(K._SIGNATURES) | set(rt_abi.SIGNATURES) | set(hyb.SIGNATURES) | set(tpm.SIGNATURES) \
        | set(bench_abi.SIGNATURES)
    declared = _declared_symbols()
    assert declared - bound == set(), f"declared but not bound in Python: {sorted(declared - bound)}"
    assert bound - declared == set(), f"bound in Python but not declared: {sorted(bound - declared)}"
    for name in bound:
        assert hasattr(lib, name), name


def test_reference_wrapper_names_present():
    """The names the reference's runtime.py imports from its kernel module (runtime.py:26-47, 123-127)."""
    for name in ["add_inplace", "has_amx", "has_batched_helpers", "has_batched_matmul", "has_fused_rmsnorm_quantize",
                 "lm_head_bf16", "lm_head_int4", "lm_head_int8", "matmul_amx_mT", "matmul_amx_mT_padded",
                 "matmul_packed_m1", "matmul_packed_mT", "quantize_activation", "quantize_activation_batched",
                 "relu2_mul_into", "relu2_mul_into_batched", "rmsnorm_into", "rmsnorm_into_batched",
                 "rmsnorm_quantize_into", "rmsnorm_quantize_batched", "matmul_unpacked_m1",
                 "matmul_accelerate_f32_m1", "has_omp", "max_threads", "has_accelerate", "ensure_built",
                 "matmul_packed_prefill", "has_unpacked_matmul"]:
        assert callable(getattr(K, name)), name
    rt = importlib.import_module("litespark_inference_b200.torchless.runtime")
    for name in ["init_state", "forward_one", "forward_prefill", "forward_prefill_all_logits", "generate",
                 "generate_speculative", "_lookup_speculation", "falcon_forward_one", "falcon_forward_prefill",
                 "falcon_generate", "InferState"]:
        assert hasattr(rt, name), name


def test_no_cpu_fallback_without_gpu():
    """Without a GPU a kernel call must fail loudly, not compute on the host."""
    lib = K.load_library(require_device=False)
    if lib.lspk_device_count() > 0:
        pytest.skip("a GPU is present")
    with pytest.raises(K.KernelUnavailable):
        K.quantize_activation(np.zeros(16, np.float32), np.zeros(16, np.int8))
    assert lib.lspk_malloc(16) is None


def test_lookup_speculation_matches_oracle(oracle):
    rt = importlib.import_module("litespark_inference_b200.torchless.runtime")
    rng = np.random.default_rng(3)
    for _ in range(200):
        ctx = [int(t) for t in rng.integers(0, 4, rng.integers(0, 24))]
        n, k = int(rng.integers(1, 6)), int(rng.integers(0, 6))
        assert rt._lookup_speculation(ctx, n, k) == oracle.lookup_speculation(ctx, n, k)
    assert rt._lookup_speculation([1, 2, 3, 9, 1, 2, 3], 4, 4) == [9, 1, 2, 3]
