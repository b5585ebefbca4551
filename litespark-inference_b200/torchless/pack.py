"""2-bit packing of ternary weights, four per byte -- the on-disk / host format.

Same format as the reference's ``litespark_inference/torchless/pack.py``: weight k of a row
is stored as ``w + 1`` in bits ``2*(k % 4)`` of byte ``k // 4``; K is padded to a multiple of
four with weight 0.  This is the INPUT format of ``lspk_upload_packed``.
"""
from __future__ import annotations

import numpy as np


def pack_ternary_4_per_byte(w_int8: np.ndarray) -> np.ndarray:
    """int8 {-1,0,+1} [N, K] -> uint8 [N, ceil(K/4)] (reference pack.py:16-45)."""
    if w_int8.dtype != np.int8 or w_int8.ndim != 2:
        raise TypeError("expected an int8 matrix")
    N, K = w_int8.shape
    Kb = (K + 3) // 4
    codes = np.full((N, Kb * 4), 1, dtype=np.uint8)
    np.add(w_int8.view(np.uint8), np.uint8(1), out=codes[:, :K], casting="unsafe")
    quads = codes.reshape(N, Kb, 4)
    out = quads[:, :, 0].copy()
    for j in (1, 2, 3):
        out |= quads[:, :, j] << np.uint8(2 * j)
    return out


def unpack_4_per_byte(w_packed: np.ndarray, K: int) -> np.ndarray:
    """uint8 [N, Kb] -> int8 {-1,0,+1} [N, K] (reference pack.py:48-62)."""
    N, Kb = w_packed.shape
    if Kb * 4 < K:
        raise ValueError("K larger than the packed row")
    out = np.empty((N, Kb, 4), dtype=np.int8)
    for j in range(4):
        out[:, :, j] = ((w_packed >> np.uint8(2 * j)) & np.uint8(3)).astype(np.int8) - 1
    return out.reshape(N, Kb * 4)[:, :K]
