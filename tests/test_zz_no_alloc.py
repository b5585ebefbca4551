"""The allocation-free GEMV entry point against the ordinary one.

``matmul_lut_sm100_m1_noalloc`` serves hosts that may not allocate GPU memory at call time -- a
serving process whose memory pool already owns the whole GPU, or a loop that has to stay clear of
the CUDA allocator -- by keeping all of its device scratch in one fixed array inside the library.
That array is shared by every call and keeps the previous call's bytes, so the test makes two
different calls in a row and requires each to equal what ``matmul_lut_sm100_m1`` returns for the
same inputs, bit for bit (the two run the same kernel on the same values).  This file sorts last on
purpose: a run that stops at the first failure has then already been through every other test.
"""
import ctypes
import importlib

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

K = importlib.import_module("litespark_inference_b200.torchless.kernel")
pack = importlib.import_module("litespark_inference_b200.torchless.pack")


def _case(seed, N, Kdim):
    rng = np.random.default_rng(seed)
    packed = pack.pack_ternary_4_per_byte(rng.integers(-1, 2, (N, Kdim), dtype=np.int8))
    xq = rng.integers(-127, 128, Kdim, dtype=np.int8)
    return packed, xq, float(np.float32(rng.uniform(0.5, 1.5))), float(np.float32(rng.uniform(0.01, 0.1)))


def test_noalloc_matches_allocating_entry_point_twice_in_a_row():
    # a large matrix first, then a smaller ragged one that lands on the first call's leftovers
    for seed, N, Kdim in ((1, 6912, 2560), (2, 33, 260), (3, 2560, 2560)):
        packed, xq, ws, xs = _case(seed, N, Kdim)
        want = K.matmul_packed_m1(xq, packed, ws, xs)
        got = K.matmul_packed_m1_noalloc(xq, packed, ws, xs)
        assert np.array_equal(got, want), f"N={N} K={Kdim}"
        again = K.matmul_packed_m1_noalloc(xq, packed, ws, xs)
        assert np.array_equal(again, want)


def _free_bytes(lib):
    free = ctypes.c_size_t(0)
    assert lib.lspk_mem_info(ctypes.byref(free), None) == 0
    return free.value


def test_noalloc_call_leaves_free_device_memory_unchanged():
    """What the entry point promises a host without an allocator: after its first call has bound the
    library, a call of any accepted size takes no device memory (cudaMemGetInfo before and after)."""
    lib = K.load_library()
    packed, xq, ws, xs = _case(6, 2560, 2560)
    K.matmul_packed_m1_noalloc(xq, packed, ws, xs)       # first call on this device: binds, looks the array up
    before = _free_bytes(lib)
    for seed, N, Kdim in ((7, 6912, 2560), (8, 640, 2560)):
        packed, xq, ws, xs = _case(seed, N, Kdim)
        K.matmul_packed_m1_noalloc(xq, packed, ws, xs)
    assert _free_bytes(lib) == before


def test_noalloc_rejects_what_does_not_fit():
    packed, xq, ws, xs = _case(4, 6912, 6912)          # about 24 MB of scratch: beyond the fixed array
    lib = K.load_library()
    lib.lspk_clear_error()
    with pytest.raises(K.KernelError, match="device scratch"):
        K.matmul_packed_m1_noalloc(xq, packed, ws, xs)
    lib.lspk_clear_error()
    # and the entry point still works afterwards
    packed, xq, ws, xs = _case(5, 640, 2560)
    assert np.array_equal(K.matmul_packed_m1_noalloc(xq, packed, ws, xs), K.matmul_packed_m1(xq, packed, ws, xs))
