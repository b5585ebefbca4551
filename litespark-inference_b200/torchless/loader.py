"""Checkpoint -> model pipeline: bf16 safetensors of a BitNet b1.58 checkpoint to the packed
ternary model the runtime runs, from a LOCAL directory (nothing is downloaded).

Follows the reference's loader (litespark_inference/torchless/loader.py:99-151 projections,
153-219 embedding quantisers, 222-355 model assembly): every linear projection is quantised with the
per-tensor absmean rule and packed four weights per byte; norms stay bf16; the tied embedding / LM
head stays bf16 or is quantised per row to int8 or int4.

Where the work happens: ``mean |W|`` is accumulated on the host in the reference's order (a float64
running sum of fp32 block sums -- the order is part of the result); with ``device_quantize=True``
(default) the ternarisation, packing and re-tiling of the projections run on the GPU straight from the
bf16 master weights (``lspk_upload_bf16_ternary``), so the host never builds the int8 or packed
copies; with ``device_quantize=False`` the host produces the reference's packed arrays (useful for the
CPU checkers, which read ``w_packed``)."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Optional

import numpy as np

from .model import BitNetConfig, PackedBitNetModel, PackedLayer, PackedProjection
from .pack import pack_ternary_4_per_byte
from .quantize import absmean_bf16, bf16_u16_to_fp32, quantize_ternary_absmean
from .safetensors_io import SafetensorsFile, open_safetensors

_PROJ_SUFFIX = {
    "q_proj": ".self_attn.q_proj.weight", "k_proj": ".self_attn.k_proj.weight",
    "v_proj": ".self_attn.v_proj.weight", "o_proj": ".self_attn.o_proj.weight",
    "gate_proj": ".mlp.gate_proj.weight", "up_proj": ".mlp.up_proj.weight",
    "down_proj": ".mlp.down_proj.weight",
}
_NORM_SUFFIX = {
    "input_norm": ".input_layernorm.weight", "post_attn_norm": ".post_attention_layernorm.weight",
    "attn_sub_norm": ".self_attn.attn_sub_norm.weight", "ffn_sub_norm": ".mlp.ffn_sub_norm.weight",
}


def config_from_hf(cfg: dict) -> BitNetConfig:
    """``config.json`` of the Hugging Face checkpoint -> BitNetConfig."""
    return BitNetConfig(hidden_size=int(cfg["hidden_size"]), num_layers=int(cfg["num_hidden_layers"]),
                        num_heads=int(cfg["num_attention_heads"]),
                        num_kv_heads=int(cfg.get("num_key_value_heads", cfg["num_attention_heads"])),
                        intermediate_size=int(cfg["intermediate_size"]), vocab_size=int(cfg["vocab_size"]),
                        max_position_embeddings=int(cfg.get("max_position_embeddings", 4096)),
                        rms_norm_eps=float(cfg.get("rms_norm_eps", 1e-5)),
                        rope_theta=float(cfg.get("rope_theta", 500000.0)))


def _bf16_bits(sf: SafetensorsFile, name: str, copy: bool) -> np.ndarray:
    a, tag = (sf.get(name) if copy else sf.view(name))
    if tag == "BF16":
        return a
    if tag == "F32":
        return (np.ascontiguousarray(a).view(np.uint32) >> 16).astype(np.uint16)
    raise ValueError(f"{name}: expected BF16 (or F32) master weights, found {tag}")


def load_projection(sf: SafetensorsFile, name: str, device_quantize: bool) -> PackedProjection:
    w = _bf16_bits(sf, name, copy=False)
    N, K = w.shape
    if K % 4:
        raise ValueError(f"{name}: in_features {K} is not a multiple of 4")
    if device_quantize:
        # keep only the bits and the scale; the GPU ternarises at upload
        return PackedProjection(w_packed=None, w_sum=None, scale=absmean_bf16(w), in_features=K, out_features=N,
                                w_bf16=w)
    t, scale = quantize_ternary_absmean(w)
    return PackedProjection(w_packed=pack_ternary_4_per_byte(t), w_sum=t.sum(axis=1, dtype=np.int32), scale=scale,
                            in_features=K, out_features=N)


def quantize_embedding(emb_u16: np.ndarray, levels: int, row_block: int = 4096):
    """Per-row absmax quantiser of the embedding table (reference loader.py:153-219): scale =
    max(|row|, 1e-5) / levels, q = clip(round(row / scale), -levels, levels).  levels = 127 gives int8
    [V, H]; levels = 7 gives int4 packed two per byte, low nibble = even column."""
    V, H = emb_u16.shape
    if levels == 7 and H % 2:
        raise ValueError(f"int4 embedding requires an even hidden size, got {H}")
    out = np.empty((V, H if levels == 127 else H // 2), dtype=np.int8 if levels == 127 else np.uint8)
    scales = np.empty(V, dtype=np.float32)
    for v0 in range(0, V, row_block):
        blk = bf16_u16_to_fp32(emb_u16[v0:v0 + row_block])
        scale = np.maximum(np.abs(blk).max(axis=1), 1e-5) / np.float32(levels)
        q = np.round(blk * (1.0 / scale)[:, None]).clip(-levels, levels).astype(np.int8)
        if levels == 127:
            out[v0:v0 + row_block] = q
        else:
            out[v0:v0 + row_block] = (q[:, 0::2].astype(np.uint8) & 0x0F) | ((q[:, 1::2].astype(np.uint8) & 0x0F) << 4)
        scales[v0:v0 + row_block] = scale
    return out, scales


def load_bitnet_dir(path, *, embed_dtype: str = "int4", device_quantize: bool = True,
                    safetensors_name: Optional[str] = None) -> PackedBitNetModel:
    """Directory with ``config.json`` and ``model.safetensors`` (bf16 master weights, Hugging Face
    tensor names) -> PackedBitNetModel.  embed_dtype: "bf16" | "int8" | "int4"."""
    if embed_dtype not in ("bf16", "int8", "int4"):
        raise ValueError("embed_dtype must be 'bf16', 'int8' or 'int4'")
    d = Path(path)
    cfg_path = d / "config.json"
    st_path = d / (safetensors_name or "model.safetensors")
    if not cfg_path.exists() or not st_path.exists():
        raise FileNotFoundError(f"{d}: need config.json and {st_path.name} (this build never downloads a checkpoint)")
    config = config_from_hf(json.loads(cfg_path.read_text()))
    sf = open_safetensors(st_path)
    emb = _bf16_bits(sf, "model.embed_tokens.weight", copy=False)
    if emb.shape != (config.vocab_size, config.hidden_size):
        raise ValueError(f"embedding shape {emb.shape} does not match the config")
    model = PackedBitNetModel(config=config, embed_tokens=None, final_norm=_bf16_bits(sf, "model.norm.weight", copy=True))
    if embed_dtype == "bf16":
        model.embed_tokens = np.array(emb)
    elif embed_dtype == "int8":
        model.embed_int8, model.embed_scale = quantize_embedding(emb, 127)
    else:
        model.embed_int4, model.embed_scale = quantize_embedding(emb, 7)
    for i in range(config.num_layers):
        prefix = f"model.layers.{i}"
        projs = {k: load_projection(sf, prefix + suf, device_quantize) for k, suf in _PROJ_SUFFIX.items()}
        norms = {k: _bf16_bits(sf, prefix + suf, copy=True) for k, suf in _NORM_SUFFIX.items()}
        model.layers.append(PackedLayer(**projs, **norms))
    if device_quantize:
        # upload now, while the mapping is alive, then drop the references to it
        from . import runtime
        runtime.to_device(model)
        for L in model.layers:
            for k in _PROJ_SUFFIX:
                getattr(L, k).w_bf16 = None
    sf.close()
    return model


def save_bitnet_dir(path, config: BitNetConfig, tensors: dict) -> None:
    """Write a checkpoint directory in the layout ``load_bitnet_dir`` reads (synthetic checkpoints, tests).
    ``tensors`` maps Hugging Face tensor names to bf16 bits (uint16 arrays)."""
    from .safetensors_io import save_safetensors
    d = Path(path)
    d.mkdir(parents=True, exist_ok=True)
    (d / "config.json").write_text(json.dumps({
        "hidden_size": config.hidden_size, "num_hidden_layers": config.num_layers,
        "num_attention_heads": config.num_heads, "num_key_value_heads": config.num_kv_heads,
        "intermediate_size": config.intermediate_size, "vocab_size": config.vocab_size,
        "max_position_embeddings": config.max_position_embeddings, "rms_norm_eps": config.rms_norm_eps,
        "rope_theta": config.rope_theta}))
    save_safetensors(d / "model.safetensors", {k: (v, "BF16") for k, v in tensors.items()})
