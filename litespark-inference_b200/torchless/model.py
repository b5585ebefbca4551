"""Plain-data containers for a packed ternary model (host side).

Field names follow ``litespark_inference/torchless/model.py`` so that code written against the
reference's containers (loaders, benchmarks) works unchanged; the reference's CPU-only
alternates (``w_float32``, ``w_unpacked``, ``w_amx``) have no counterpart here.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

import numpy as np


@dataclass
class BitNetConfig:
    hidden_size: int
    num_layers: int
    num_heads: int
    num_kv_heads: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float


@dataclass
class PackedProjection:
    """One ternary projection: uint8 [N, ceil(K/4)] packed weights + per-tensor scale
    (reference model.py:26-49)."""
    w_packed: Optional[np.ndarray]
    w_sum: Optional[np.ndarray]
    scale: float
    in_features: int
    out_features: int
    # bf16 master weights (uint16 bits, [N, K]) of a projection that is ternarised on the device at
    # upload instead of on the host: w_packed is then None and scale is mean |W| as a Python float
    w_bf16: Optional[np.ndarray] = None


@dataclass
class PackedLayer:
    q_proj: PackedProjection
    k_proj: PackedProjection
    v_proj: PackedProjection
    o_proj: PackedProjection
    gate_proj: PackedProjection
    up_proj: PackedProjection
    down_proj: PackedProjection
    input_norm: np.ndarray          # bf16 bits (uint16) or fp32
    post_attn_norm: np.ndarray
    attn_sub_norm: Optional[np.ndarray] = None   # BitNet only
    ffn_sub_norm: Optional[np.ndarray] = None


@dataclass
class PackedBitNetModel:
    config: BitNetConfig
    embed_tokens: Optional[np.ndarray]           # bf16 bits [V, H] or None when quantised
    final_norm: np.ndarray
    projection_backend: str = "sm100"
    layers: list = field(default_factory=list)
    embed_int8: Optional[np.ndarray] = None      # int8 [V, H]
    embed_scale: Optional[np.ndarray] = None     # fp32 [V]
    embed_int4: Optional[np.ndarray] = None      # uint8 [V, H/2], low nibble first

    def tensor_bytes(self) -> dict:
        """Stored bytes by category (reference model.py:123-163)."""
        nb = lambda a: int(a.nbytes) if isinstance(a, np.ndarray) else 0
        packed = norms = 0
        for L in self.layers:
            for name in ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"):
                packed += nb(getattr(L, name).w_packed)
            for name in ("input_norm", "post_attn_norm", "attn_sub_norm", "ffn_sub_norm"):
                norms += nb(getattr(L, name))
        emb = nb(self.embed_tokens) + nb(self.embed_int8) + nb(self.embed_int4) + nb(self.embed_scale)
        rest = packed + norms + nb(self.final_norm)
        return {"packed_weights": packed, "per_layer_norms": norms, "final_norm": nb(self.final_norm),
                "embedding": emb, "total_excl_embedding": rest, "total_incl_embedding": rest + emb}


@dataclass
class FalconTernaryConfig(BitNetConfig):
    eos_token_ids: Tuple[int, ...] = (2,)


@dataclass
class PackedFalconLayer:
    """One Falcon-E layer (reference model.py:180-189): no sub-norms."""
    q_proj: PackedProjection
    k_proj: PackedProjection
    v_proj: PackedProjection
    o_proj: PackedProjection
    gate_proj: PackedProjection
    up_proj: PackedProjection
    down_proj: PackedProjection
    input_norm: np.ndarray
    post_attn_norm: np.ndarray
    attn_sub_norm: None = None      # read by the uploader, which treats both families alike
    ffn_sub_norm: None = None


@dataclass
class PackedFalconModel:
    """Falcon-E family (reference model.py:166-250): SiLU gate, no sub-norms, untied LM head."""
    config: FalconTernaryConfig
    embed_tokens: Optional[np.ndarray]
    final_norm: np.ndarray
    projection_backend: str = "sm100"
    layers: list = field(default_factory=list)
    embed_int8: Optional[np.ndarray] = None
    embed_int4: Optional[np.ndarray] = None
    embed_scale: Optional[np.ndarray] = None
    lm_head_tokens: Optional[np.ndarray] = None
    lm_head_int8: Optional[np.ndarray] = None
    lm_head_int4: Optional[np.ndarray] = None
    lm_head_scale: Optional[np.ndarray] = None
