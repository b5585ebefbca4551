"""Row-split tensor parallelism of the MLP projections (optional; the reference has none).

Host-side logic shared by both transports:

* ``split_rows`` / ``slice_projection``: rank r of g gets output rows ``[r*N/g, (r+1)*N/g)`` of a
  packed matrix (packed rows are independent, so a slice is a plain row range of the packed bytes).
* ``mlp_block``: gate/up slice -> ReLU^2 gate -> all-gather -> SubLN + quantiser -> down slice ->
  all-gather.  The ``compute`` and ``gather`` steps are supplied by the transport:
  - ``DeviceTP``: the CUDA kernels + NCCL all-gather over NVLink (``include/lspk_tp.h``);
  - ``HostGroup``: any object with ``all_gather(np.ndarray) -> np.ndarray`` (the CPU tests pass a
    torch.distributed/gloo wrapper and use the CPU oracle as the compute), which exercises the
    partitioning logic with world_size > 1 and no GPU.
"""
from __future__ import annotations

import ctypes
from typing import Callable, Optional

import numpy as np

from . import kernel as _k
from .model import PackedProjection

_ci, _cf, _vp, _sz = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t

SIGNATURES = {
    "lspk_tp_unique_id": ([_vp], _ci),
    "lspk_tp_init": ([_vp, _ci, _ci], _ci),
    "lspk_tp_rank": ([], _ci),
    "lspk_tp_world": ([], _ci),
    "lspk_tp_allgather_f32": ([_vp, _vp, _sz], _ci),
    "lspk_tp_finalize": ([], _ci),
    "lspk_tp_window_create": ([_ci, _ci, _ci, _ci, _vp], _ci),
    "lspk_tp_window_open": ([_ci, _vp], _ci),
    "lspk_tp_window_close": ([], _ci),
    "lspk_tp_window_set_poll_limit": ([ctypes.c_uint], _ci),
    "lspk_tp_window_vector": ([_ci], _vp),
    "lspk_tp_debug_drop_next_arrival": ([], _ci),
    "lspk_tp_exchange": ([_vp, _ci], _ci),
    "lspk_tp_mlp_block_peer": ([_vp, _vp, _vp, _vp, _vp, _vp, _cf, _vp, _vp], _ci),
    "lspk_tp_mlp_block": ([_vp, _vp, _vp, _vp, _vp, _vp, _cf, _vp, _vp, _vp, _vp], _ci),
}


def _lib():
    lib = _k.load_library(True)
    if not getattr(lib, "_tp_bound", False):
        for name, (argtypes, restype) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = restype
        lib._tp_bound = True
    return lib


def row_range(N: int, world: int, rank: int):
    """Rows of rank `rank`: equal slices; N must divide evenly (it does for 6912 and 2560 at g = 2, 4, 8)."""
    if N % world:
        raise ValueError(f"N={N} is not divisible by the tensor-parallel degree {world}")
    n = N // world
    return rank * n, (rank + 1) * n


def slice_projection(p: PackedProjection, world: int, rank: int) -> PackedProjection:
    lo, hi = row_range(p.out_features, world, rank)
    return PackedProjection(w_packed=np.ascontiguousarray(p.w_packed[lo:hi]), w_sum=None, scale=p.scale,
                            in_features=p.in_features, out_features=hi - lo)


def mlp_block(x: np.ndarray, layer, eps: float, world: int, rank: int,
              gate_up_slice: Callable, down_slice: Callable, all_gather: Callable) -> np.ndarray:
    """The row-split MLP block on host arrays.  ``gate_up_slice(x)`` returns this rank's slice of
    relu(gate h)^2 * (up h); ``down_slice(inter)`` this rank's slice of the down projection;
    ``all_gather(v)`` the concatenation over ranks in rank order.  Returns the full down output."""
    inter = all_gather(gate_up_slice(x))
    return all_gather(down_slice(inter))


class DeviceTP:
    """NCCL transport + CUDA compute for one rank (one process per GPU)."""

    def __init__(self, rank: int, world: int, unique_id: Optional[bytes] = None):
        self.lib = _lib()
        self.rank, self.world = rank, world
        if world > 1:
            assert unique_id is not None and len(unique_id) == 128
            buf = ctypes.create_string_buffer(unique_id, 128)
            _k.check(self.lib.lspk_tp_init(buf, rank, world))

    @staticmethod
    def make_unique_id() -> bytes:
        buf = ctypes.create_string_buffer(128)
        _k.check(_lib().lspk_tp_unique_id(buf))
        return buf.raw

    def all_gather(self, send, recv, count_per_rank: int) -> None:
        _k.check(self.lib.lspk_tp_allgather_f32(send.ptr, recv.ptr, count_per_rank))

    def mlp_block(self, gate_r, up_r, down_r, x, norm, sub_norm, eps, inter_slice, inter_full, down_slice, y_full):
        _k.check(self.lib.lspk_tp_mlp_block(gate_r.handle, up_r.handle, down_r.handle, x.ptr, norm.ptr, sub_norm.ptr,
                                            eps, inter_slice.ptr, inter_full.ptr, down_slice.ptr, y_full.ptr))

    # ---- exchange over peer memory (CUDA IPC windows) instead of NCCL -------------------------------------------
    def create_window(self, I: int, H: int) -> bytes:
        """Allocate this rank's window for gathered vectors of I and H floats; returns its 64-byte IPC handle,
        which the caller passes to every other rank (any host channel)."""
        buf = ctypes.create_string_buffer(64)
        _k.check(self.lib.lspk_tp_window_create(self.rank, self.world, I, H, buf))
        self._window = (I, H)
        return buf.raw

    def open_windows(self, handles) -> None:
        """handles[r] = the 64-byte handle rank r created (this rank's own entry is ignored)."""
        for r, h in enumerate(handles):
            if r != self.rank:
                _k.check(self.lib.lspk_tp_window_open(r, ctypes.create_string_buffer(bytes(h), 64)))

    def mlp_block_peer(self, gate_r, up_r, down_r, x, norm, sub_norm, eps, inter_slice, down_slice) -> np.ndarray:
        """The row-split MLP block with both gathers through the windows; returns the gathered down product."""
        _k.check(self.lib.lspk_tp_mlp_block_peer(gate_r.handle, up_r.handle, down_r.handle, x.ptr, norm.ptr, sub_norm.ptr,
                                                 eps, inter_slice.ptr, down_slice.ptr))
        return self.window_vector(1)

    def window_vector(self, which: int) -> np.ndarray:
        n = self._window[which]
        out = np.empty(n, np.float32)
        _k.check(self.lib.lspk_d2h(out.ctypes.data, self.lib.lspk_tp_window_vector(which), out.nbytes))
        return out

    def close_window(self) -> None:
        self.lib.lspk_tp_window_close()

    def close(self):
        self.lib.lspk_tp_window_close()
        self.lib.lspk_tp_finalize()
