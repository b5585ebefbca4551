"""Host-side numpy pieces the device runtime still needs: the RoPE tables.

The tables are computed on the host exactly as the reference does
(``litespark_inference/torchless/ops.py:40-50``: fp32 inverse frequencies, fp32 angles) and
uploaded once per inference state, so the rotation on the GPU uses bit-identical cos / sin.
"""
from __future__ import annotations

import numpy as np


def rope_tables(head_dim: int, max_pos: int, theta: float):
    """(cos, sin), each fp32 [max_pos, head_dim / 2]."""
    inv_freq = 1.0 / (theta ** (np.arange(0, head_dim, 2, dtype=np.float32) / head_dim))
    freqs = np.arange(max_pos, dtype=np.float32)[:, None] * inv_freq[None, :]
    return np.cos(freqs).astype(np.float32), np.sin(freqs).astype(np.float32)
