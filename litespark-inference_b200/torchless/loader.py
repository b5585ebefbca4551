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

from .model import (BitNetConfig, FalconTernaryConfig, PackedBitNetModel, PackedFalconLayer, PackedFalconModel,
                    PackedLayer, PackedProjection)
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


# ---- Falcon-E family: checkpoints that already hold ternary weights in the Hugging Face packing ---------------
def unpack_hf_packed_bitnet(packed: np.ndarray, out_features: int) -> np.ndarray:
    """Hugging Face BitNet packing -> int8 {-1, 0, +1} [out_features, K] (reference loader.py:381-390).
    The checkpoint stores uint8 [ceil(N / 4), K]: byte (r, c) carries, in its bit pairs 0..3, column c of rows
    r, r + n, r + 2n, r + 3n (n = number of byte rows), each as weight + 1."""
    if packed.ndim == 1:
        packed = packed[:, None]
    n, cols = packed.shape
    out = np.empty((4 * n, cols), dtype=np.uint8)
    for i in range(4):
        out[i * n:(i + 1) * n] = (packed >> (2 * i)) & 0x3
    return out[:out_features].astype(np.int8) - 1


def load_falcon_projection(sf: SafetensorsFile, key: str, out_features: int) -> PackedProjection:
    """One packed projection of a Falcon-E checkpoint (reference loader.py:393-434): re-packed along K into
    the reference's four-weights-per-byte rows; the per-tensor scale is the reciprocal of the stored
    ``<key>_scale`` tensor (1 when absent)."""
    raw, tag = sf.get(key)
    if raw.dtype != np.uint8:
        raise ValueError(f"expected packed uint8 Falcon projection {key}, got {tag}")
    t = unpack_hf_packed_bitnet(raw, out_features)
    scale = 1.0
    if key + "_scale" in sf:
        sc, sc_tag = sf.get(key + "_scale")
        sc32 = bf16_u16_to_fp32(sc) if sc_tag == "BF16" else sc.astype(np.float32)
        scale = float(1.0 / sc32.reshape(-1)[0])
    N, K = t.shape
    if K % 4:
        raise ValueError(f"{key}: in_features {K} is not a multiple of 4")
    return PackedProjection(w_packed=pack_ternary_4_per_byte(t), w_sum=t.sum(axis=1, dtype=np.int32), scale=scale,
                            in_features=K, out_features=N)


def _dense_table(sf: SafetensorsFile, key: str, embed_dtype: str):
    """bf16 [V, H] table -> (bf16, int8, int4, scale), one of the first three set (reference loader.py:437-450)."""
    raw, tag = sf.view(key)
    if tag != "BF16":
        raise ValueError(f"Falcon dense tensor {key} must be BF16, got {tag}")
    if embed_dtype == "bf16":
        return np.array(raw), None, None, None
    if embed_dtype == "int8":
        q, sc = quantize_embedding(raw, 127)
        return None, q, None, sc
    q, sc = quantize_embedding(raw, 7)
    return None, None, q, sc


def load_falcon_dir(path, *, embed_dtype: str = "int4", safetensors_name: Optional[str] = None) -> PackedFalconModel:
    """Directory with ``config.json`` and ``model.safetensors`` of a Falcon-E checkpoint (projections already
    ternary in the Hugging Face packing, bf16 norms, bf16 embedding and -- when present -- untied ``lm_head``)
    -> PackedFalconModel, following the reference's load_falcon_edge (loader.py:453-536) minus the download."""
    if embed_dtype not in ("bf16", "int8", "int4"):
        raise ValueError("embed_dtype must be 'bf16', 'int8' or 'int4'")
    d = Path(path)
    cfg_path, st_path = d / "config.json", d / (safetensors_name or "model.safetensors")
    if not cfg_path.exists() or not st_path.exists():
        raise FileNotFoundError(f"{d}: need config.json and {st_path.name} (this build never downloads a checkpoint)")
    hf = json.loads(cfg_path.read_text())
    eos = hf.get("eos_token_id", 2)
    config = FalconTernaryConfig(
        hidden_size=int(hf["hidden_size"]), num_layers=int(hf["num_hidden_layers"]),
        num_heads=int(hf["num_attention_heads"]),
        num_kv_heads=int(hf.get("num_key_value_heads", hf["num_attention_heads"])),
        intermediate_size=int(hf["intermediate_size"]), vocab_size=int(hf["vocab_size"]),
        max_position_embeddings=int(hf.get("max_position_embeddings", 2048)),
        rms_norm_eps=float(hf.get("rms_norm_eps", 1e-5)), rope_theta=float(hf.get("rope_theta", 10000.0)),
        eos_token_ids=tuple(eos) if isinstance(eos, list) else (int(eos),))
    sf = open_safetensors(st_path)
    try:
        e16, e8, e4, esc = _dense_table(sf, "model.embed_tokens.weight", embed_dtype)
        if "lm_head.weight" in sf:
            l16, l8, l4, lsc = _dense_table(sf, "lm_head.weight", embed_dtype)
        else:
            l16, l8, l4, lsc = e16, e8, e4, esc
        kv_out = config.num_kv_heads * (config.hidden_size // config.num_heads)
        rows = {"q_proj": config.hidden_size, "k_proj": kv_out, "v_proj": kv_out, "o_proj": config.hidden_size,
                "gate_proj": config.intermediate_size, "up_proj": config.intermediate_size,
                "down_proj": config.hidden_size}
        layers = []
        for i in range(config.num_layers):
            prefix = f"model.layers.{i}"
            projs = {k: load_falcon_projection(sf, prefix + suf, rows[k]) for k, suf in _PROJ_SUFFIX.items()}
            layers.append(PackedFalconLayer(
                **projs, input_norm=_bf16_bits(sf, prefix + _NORM_SUFFIX["input_norm"], copy=True),
                post_attn_norm=_bf16_bits(sf, prefix + _NORM_SUFFIX["post_attn_norm"], copy=True)))
        return PackedFalconModel(config=config, embed_tokens=e16, final_norm=_bf16_bits(sf, "model.norm.weight", copy=True),
                                 layers=layers, embed_int8=e8, embed_int4=e4, embed_scale=esc, lm_head_tokens=l16,
                                 lm_head_int8=l8, lm_head_int4=l4, lm_head_scale=lsc)
    finally:
        sf.close()


def save_falcon_dir(path, config: FalconTernaryConfig, tensors: dict) -> None:
    """Write a Falcon-E checkpoint directory in the layout ``load_falcon_dir`` reads (synthetic checkpoints,
    tests).  ``tensors`` maps tensor names to (array, safetensors dtype tag)."""
    from .safetensors_io import save_safetensors
    d = Path(path)
    d.mkdir(parents=True, exist_ok=True)
    (d / "config.json").write_text(json.dumps({
        "hidden_size": config.hidden_size, "num_hidden_layers": config.num_layers,
        "num_attention_heads": config.num_heads, "num_key_value_heads": config.num_kv_heads,
        "intermediate_size": config.intermediate_size, "vocab_size": config.vocab_size,
        "max_position_embeddings": config.max_position_embeddings, "rms_norm_eps": config.rms_norm_eps,
        "rope_theta": config.rope_theta, "eos_token_id": list(config.eos_token_ids)}))
    save_safetensors(d / "model.safetensors", tensors)


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
