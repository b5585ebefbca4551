"""Hybrid Mamba-2 + ternary-MoE decoder: host containers, seeded synthetic generator and the
device runtime (``include/lspk_hybrid.h``).

The reference has no such blocks; shapes and initial distributions follow the benchmark
configuration: 24 layers alternating Mamba-2 and MoE at hidden 2560; Mamba-2 with 80 heads x 64,
d_state 128, one group, conv width 4, ``A = -exp(U(-4, 0))``, ``dt_bias ~ U(-4, -2)``, ternary in/out
projections; MoE with 8 ternary experts of FFN width 6912 and squared ReLU stored as ONE packed
buffer, top-2 fp32 softmax router ``~ N(0, 0.02)``.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np

from . import kernel as _k
from .model import PackedProjection
from .quantize import fp32_to_bf16_u16
from .synthetic import random_projection, random_projection_fast

_ci, _cf, _vp, _sz = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t


class MambaConfigC(ctypes.Structure):
    """Mirror of ``lspk_mamba_config``."""
    _fields_ = [("hidden", _ci), ("nheads", _ci), ("headdim", _ci), ("d_state", _ci), ("conv_width", _ci),
                ("eps", _cf)]


SIGNATURES = {
    "lspk_moe_create": ([_ci, _ci, _ci, _vp, _vp, _vp, _vp, _vp, _cf], _vp),
    "lspk_moe_free": ([_vp], _ci),
    "lspk_moe_device_bytes": ([_vp], _sz),
    "lspk_moe_forward": ([_vp, _vp, _ci, _vp, _vp, _vp, _vp, _vp], _ci),
    "lspk_mamba_create": ([ctypes.POINTER(MambaConfigC), _vp, _cf, _vp, _cf, _vp, _vp, _vp, _vp, _vp, _vp, _vp], _vp),
    "lspk_mamba_free": ([_vp], _ci),
    "lspk_mamba_device_bytes": ([_vp], _sz),
    "lspk_mamba_state_floats": ([_vp], _sz),
    "lspk_mamba_step": ([_vp, _vp, _vp, _vp, _ci], _ci),
    "lspk_hybrid_create": ([_ci, _ci, _cf], _vp),
    "lspk_hybrid_add_mamba": ([_vp, _vp], _ci),
    "lspk_hybrid_add_moe": ([_vp, _vp], _ci),
    "lspk_hybrid_set_embedding": ([_vp, _vp, _vp], _ci),
    "lspk_hybrid_free": ([_vp], _ci),
    "lspk_hybrid_device_bytes": ([_vp], _sz),
    "lspk_hybrid_state_create": ([_vp, _ci, _ci], _vp),
    "lspk_hybrid_state_free": ([_vp], _ci),
    "lspk_hybrid_state_reset": ([_vp], _ci),
    "lspk_hybrid_step": ([_vp, _vp, _vp, _vp], _ci),
    "lspk_hybrid_decode_greedy": ([_vp, _vp, _ci, _vp], _ci),
    "lspk_hybrid_prefill": ([_vp, _vp, _ci, _vp], _ci),
    "lspk_hybrid_step_kernel_count": ([_vp], _ci),
}


def _lib():
    lib = _k.load_library(True)
    if not getattr(lib, "_hybrid_bound", False):
        for name, (argtypes, restype) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = restype
        lib._hybrid_bound = True
    return lib


def _p(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


@dataclass
class HybridConfig:
    hidden_size: int = 2560
    num_layers: int = 24
    vocab_size: int = 128256
    rms_norm_eps: float = 1e-5
    # MoE
    num_experts: int = 8
    intermediate_size: int = 6912
    # Mamba-2
    nheads: int = 80
    headdim: int = 64
    d_state: int = 128
    conv_width: int = 4


@dataclass
class MoELayer:
    kind: str
    norm: np.ndarray                # bf16 [H]
    router: np.ndarray              # fp32 [E, H]
    experts_packed: np.ndarray      # uint8 [E, 3, I*H/4]: gate, up, down of each expert
    scales: np.ndarray              # fp32 [E, 3]
    sub_norm: np.ndarray            # bf16 [E, I]
    hidden_size: int
    intermediate_size: int

    def gate(self, e: int) -> np.ndarray:
        return self.experts_packed[e, 0].reshape(self.intermediate_size, self.hidden_size // 4)

    def up(self, e: int) -> np.ndarray:
        return self.experts_packed[e, 1].reshape(self.intermediate_size, self.hidden_size // 4)

    def down(self, e: int) -> np.ndarray:
        return self.experts_packed[e, 2].reshape(self.hidden_size, self.intermediate_size // 4)


@dataclass
class MambaLayer:
    kind: str
    norm: np.ndarray                # bf16 [H]
    in_proj: PackedProjection       # [2*d_inner + 2*d_state + nheads, H]
    out_proj: PackedProjection      # [H, d_inner]
    conv_w: np.ndarray              # fp32 [conv_dim, 4]
    conv_b: np.ndarray              # fp32 [conv_dim]
    A: np.ndarray                   # fp32 [nheads], negative
    dt_bias: np.ndarray             # fp32 [nheads]
    D: np.ndarray                   # fp32 [nheads]
    gated_norm: np.ndarray          # bf16 [d_inner]
    nheads: int
    headdim: int
    d_state: int

    @property
    def d_inner(self) -> int:
        return self.nheads * self.headdim

    @property
    def conv_dim(self) -> int:
        return self.d_inner + 2 * self.d_state


@dataclass
class HybridModel:
    config: HybridConfig
    embed_tokens: np.ndarray        # bf16 [V, H]
    final_norm: np.ndarray          # bf16 [H]
    layers: List = field(default_factory=list)


def random_hybrid(cfg: HybridConfig, seed: int = 0, fast: bool = False, norm_jitter: float = 0.0) -> HybridModel:
    rng = np.random.default_rng(seed)
    H, I, E = cfg.hidden_size, cfg.intermediate_size, cfg.num_experts
    proj = random_projection_fast if fast else random_projection
    di = cfg.nheads * cfg.headdim
    conv_dim = di + 2 * cfg.d_state
    in_out = 2 * di + 2 * cfg.d_state + cfg.nheads

    def gamma(*shape):
        g = np.ones(shape, dtype=np.float32)
        if norm_jitter:
            g += rng.uniform(-norm_jitter, norm_jitter, shape).astype(np.float32)
        return fp32_to_bf16_u16(g)

    layers = []
    for li in range(cfg.num_layers):
        if li % 2 == 0:
            layers.append(MambaLayer(
                kind="mamba", norm=gamma(H), in_proj=proj(rng, in_out, H), out_proj=proj(rng, H, di),
                conv_w=rng.uniform(-0.5, 0.5, (conv_dim, cfg.conv_width)).astype(np.float32),
                conv_b=rng.uniform(-0.1, 0.1, conv_dim).astype(np.float32),
                A=(-np.exp(rng.uniform(-4.0, 0.0, cfg.nheads))).astype(np.float32),
                dt_bias=rng.uniform(-4.0, -2.0, cfg.nheads).astype(np.float32),
                D=np.ones(cfg.nheads, dtype=np.float32), gated_norm=gamma(di),
                nheads=cfg.nheads, headdim=cfg.headdim, d_state=cfg.d_state))
        else:
            packed = np.empty((E, 3, I * H // 4), dtype=np.uint8)
            scales = np.empty((E, 3), dtype=np.float32)
            for e in range(E):
                for j, (n, k) in enumerate(((I, H), (I, H), (H, I))):
                    pr = proj(rng, n, k)
                    packed[e, j] = pr.w_packed.reshape(-1)
                    scales[e, j] = np.float32(pr.scale)
            layers.append(MoELayer(
                kind="moe", norm=gamma(H), router=(rng.standard_normal((E, H)) * 0.02).astype(np.float32),
                experts_packed=packed, scales=scales, sub_norm=gamma(E, I), hidden_size=H, intermediate_size=I))
    emb = np.empty((cfg.vocab_size, H), dtype=np.uint16)
    for r in range(0, cfg.vocab_size, 8192):
        n = min(8192, cfg.vocab_size - r)
        emb[r:r + n] = fp32_to_bf16_u16(rng.standard_normal((n, H), dtype=np.float32))
    return HybridModel(config=cfg, embed_tokens=emb, final_norm=gamma(H), layers=layers)


# ---- device objects -----------------------------------------------------------------------------
class DeviceMoE:
    def __init__(self, layer: MoELayer, eps: float):
        self.lib = _lib()
        E = layer.experts_packed.shape[0]
        self.layer = layer
        self.handle = self.lib.lspk_moe_create(
            E, layer.hidden_size, layer.intermediate_size, _p(np.ascontiguousarray(layer.experts_packed)),
            _p(np.ascontiguousarray(layer.scales)), _p(np.ascontiguousarray(layer.router)),
            _p(np.ascontiguousarray(layer.norm)), _p(np.ascontiguousarray(layer.sub_norm)), eps)
        if not self.handle:
            raise _k.KernelError(_k.last_error())
        self.owned = True

    def forward(self, x_dev, B: int, sel=None, selw=None, acc_gate=None, acc_up=None, acc_down=None):
        g = lambda a: a.ptr if a is not None else None
        _k.check(self.lib.lspk_moe_forward(self.handle, x_dev.ptr, B, g(sel), g(selw), g(acc_gate), g(acc_up),
                                           g(acc_down)))

    def free(self):
        if self.handle and self.owned:
            self.lib.lspk_moe_free(self.handle)
        self.handle = None


class DeviceMamba:
    def __init__(self, layer: MambaLayer, hidden: int, eps: float):
        self.lib = _lib()
        cfg = MambaConfigC(hidden, layer.nheads, layer.headdim, layer.d_state, layer.conv_w.shape[1], eps)
        c = np.ascontiguousarray
        self.handle = self.lib.lspk_mamba_create(
            ctypes.byref(cfg), _p(c(layer.in_proj.w_packed)), float(np.float32(layer.in_proj.scale)),
            _p(c(layer.out_proj.w_packed)), float(np.float32(layer.out_proj.scale)), _p(c(layer.conv_w)),
            _p(c(layer.conv_b)), _p(c(layer.A)), _p(c(layer.dt_bias)), _p(c(layer.D)), _p(c(layer.norm)),
            _p(c(layer.gated_norm)))
        if not self.handle:
            raise _k.KernelError(_k.last_error())
        self.owned = True

    @property
    def state_floats(self) -> int:
        return int(self.lib.lspk_mamba_state_floats(self.handle))

    def step(self, x_dev, state_dev, pos_dev, B: int):
        _k.check(self.lib.lspk_mamba_step(self.handle, x_dev.ptr, state_dev.ptr, pos_dev.ptr, B))

    def free(self):
        if self.handle and self.owned:
            self.lib.lspk_mamba_free(self.handle)
        self.handle = None


class DeviceHybrid:
    """GPU-resident hybrid model; owns its layers."""

    def __init__(self, model: HybridModel):
        self.lib = _lib()
        c = model.config
        self.config = c
        self.handle = self.lib.lspk_hybrid_create(c.hidden_size, c.vocab_size, c.rms_norm_eps)
        if not self.handle:
            raise _k.KernelError(_k.last_error())
        for L in model.layers:
            if L.kind == "mamba":
                d = DeviceMamba(L, c.hidden_size, c.rms_norm_eps)
                d.owned = False
                _k.check(self.lib.lspk_hybrid_add_mamba(self.handle, d.handle))
            else:
                d = DeviceMoE(L, c.rms_norm_eps)
                d.owned = False
                _k.check(self.lib.lspk_hybrid_add_moe(self.handle, d.handle))
        _k.check(self.lib.lspk_hybrid_set_embedding(self.handle, _p(np.ascontiguousarray(model.embed_tokens)),
                                                    _p(np.ascontiguousarray(model.final_norm))))

    @property
    def device_bytes(self) -> int:
        return int(self.lib.lspk_hybrid_device_bytes(self.handle))

    def close(self):
        if getattr(self, "handle", None):
            self.lib.lspk_hybrid_free(self.handle)
            self.handle = None


class HybridState:
    def __init__(self, dev: DeviceHybrid, batch: int = 1, max_steps: int = 256):
        self.dev, self.lib, self.batch, self.max_steps = dev, dev.lib, batch, max_steps
        self.handle = self.lib.lspk_hybrid_state_create(dev.handle, batch, max_steps)
        if not self.handle:
            raise _k.KernelError(_k.last_error())

    def reset(self):
        _k.check(self.lib.lspk_hybrid_state_reset(self.handle))

    def step(self, tokens, want_logits: bool = False):
        tok = np.ascontiguousarray(tokens, dtype=np.int32).reshape(self.batch)
        nxt = np.empty(self.batch, np.int32)
        logits = np.empty((self.batch, self.dev.config.vocab_size), np.float32) if want_logits else None
        _k.check(self.lib.lspk_hybrid_step(self.handle, _p(tok), _p(logits), _p(nxt)))
        return (nxt, logits) if want_logits else nxt

    def prefill(self, tokens_tb):
        tok = np.ascontiguousarray(tokens_tb, dtype=np.int32).reshape(-1, self.batch)
        nxt = np.empty(self.batch, np.int32)
        _k.check(self.lib.lspk_hybrid_prefill(self.handle, _p(tok), tok.shape[0], _p(nxt)))
        return nxt

    def decode_greedy(self, first_tokens, n_steps: int):
        first = np.ascontiguousarray(first_tokens, dtype=np.int32).reshape(self.batch)
        out = np.empty((n_steps, self.batch), np.int32)
        _k.check(self.lib.lspk_hybrid_decode_greedy(self.handle, _p(first), n_steps, _p(out)))
        return out

    @property
    def step_kernel_count(self) -> int:
        return int(self.lib.lspk_hybrid_step_kernel_count(self.handle))

    def close(self):
        if getattr(self, "handle", None):
            self.lib.lspk_hybrid_state_free(self.handle)
            self.handle = None


def generate(dev: DeviceHybrid, prompts, max_new_tokens: int):
    """Greedy decode of equally long prompts (one per sequence) in lock step; returns [B][max_new_tokens]."""
    prompts = np.ascontiguousarray(prompts, dtype=np.int32)
    if prompts.ndim == 1:
        prompts = prompts[None, :]
    B, T = prompts.shape
    st = HybridState(dev, batch=B, max_steps=max(max_new_tokens, 1))
    first = st.prefill(prompts.T)
    out = [first]
    if max_new_tokens > 1:
        out.extend(st.decode_greedy(first, max_new_tokens - 1))
    st.close()
    return np.stack(out, axis=1).tolist()
