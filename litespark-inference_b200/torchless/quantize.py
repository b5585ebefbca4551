"""Per-tensor absmean ternary quantiser and bf16 <-> fp32 bit helpers (host side, numpy).

Mirrors ``litespark_inference/torchless/quantize.py``; defines the per-tensor ``scale`` that
the kernels multiply back in.
"""
from __future__ import annotations

import numpy as np


def bf16_u16_to_fp32(a_u16: np.ndarray) -> np.ndarray:
    """bf16 bits stored as uint16 -> fp32, exact (reference quantize.py:19-21)."""
    return (a_u16.astype(np.uint32) << 16).view(np.float32)


def fp32_to_bf16_u16(a_f32: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bits by truncation (for building synthetic bf16 tensors)."""
    return (np.ascontiguousarray(a_f32, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)


def absmean_bf16(w_bf16_u16: np.ndarray, row_block: int = 128) -> float:
    """mean |W| exactly as the reference accumulates it (quantize.py:38-46): fp32 sums of blocks of
    ``row_block`` rows, added up in float64; 1.0 for an all-zero matrix."""
    if w_bf16_u16.dtype != np.uint16:
        raise TypeError("expected bf16 bits as uint16")
    N, K = w_bf16_u16.shape
    acc = 0.0
    for r in range(0, N, row_block):
        acc += float(np.abs(bf16_u16_to_fp32(w_bf16_u16[r:r + row_block])).sum())
    absmean = acc / (N * K)
    return absmean if absmean > 0.0 else 1.0


def quantize_ternary_absmean(w_bf16_u16: np.ndarray, row_block: int = 128):
    """bf16 [N, K] -> (int8 {-1,0,+1} [N, K], scale) with scale = mean |W|
    (reference quantize.py:24-60: float64 running sum of fp32 block sums, then
    round(W * (1/scale)) clipped to [-1, 1])."""
    N, K = w_bf16_u16.shape
    absmean = absmean_bf16(w_bf16_u16, row_block)
    inv = 1.0 / absmean
    w = np.empty((N, K), dtype=np.int8)
    for r in range(0, N, row_block):
        blk = bf16_u16_to_fp32(w_bf16_u16[r:r + row_block])
        w[r:r + row_block] = np.round(blk * inv).clip(-1, 1).astype(np.int8)
    return w, absmean
