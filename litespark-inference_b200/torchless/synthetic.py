"""Seeded synthetic models and inputs with the reference benchmark's shapes and value
distributions (ternary weights uniform over {-1,0,+1}, per-tensor scale ~U(0.5,1.5), norm
weights 1, bf16 embedding ~N(0,1), uniform random token ids).  They stand in for the real
checkpoint and prompt, which need network access."""
from __future__ import annotations

import numpy as np

from .model import (BitNetConfig, FalconTernaryConfig, PackedBitNetModel, PackedFalconLayer, PackedFalconModel,
                    PackedLayer, PackedProjection)
from .pack import pack_ternary_4_per_byte
from .quantize import fp32_to_bf16_u16

BITNET_2B = dict(hidden_size=2560, num_layers=30, num_heads=20, num_kv_heads=5, intermediate_size=6912,
                 vocab_size=128256, max_position_embeddings=4096, rms_norm_eps=1e-5, rope_theta=500000.0)

# (N, K) of the BitNet-2B projections
BITNET_2B_SHAPES = {"q": (2560, 2560), "k": (640, 2560), "v": (640, 2560), "o": (2560, 2560),
                    "gate": (6912, 2560), "up": (6912, 2560), "down": (2560, 6912)}


def random_projection(rng: np.random.Generator, N: int, K: int) -> PackedProjection:
    w = rng.integers(-1, 2, size=(N, K), dtype=np.int8)
    scale = float(np.float32(rng.uniform(0.5, 1.5)))
    return PackedProjection(w_packed=pack_ternary_4_per_byte(w), w_sum=None, scale=scale,
                            in_features=K, out_features=N)


# all 81 bytes that encode four trits, indexed by the base-3 number of the four codes
_TRIT_BYTES = np.array([(a) | (b << 2) | (c << 4) | (d << 6)
                        for d in range(3) for c in range(3) for b in range(3) for a in range(3)], dtype=np.uint8)


def random_projection_fast(rng: np.random.Generator, N: int, K: int) -> PackedProjection:
    """Same distribution as random_projection (i.i.d. uniform ternary weights), drawn directly as
    packed bytes: a uniform draw among the 81 four-trit bytes is four independent uniform trits.
    Several times faster, for full-size models."""
    assert K % 4 == 0
    packed = _TRIT_BYTES[rng.integers(0, 81, size=(N, K // 4), dtype=np.uint8)]
    scale = float(np.float32(rng.uniform(0.5, 1.5)))
    return PackedProjection(w_packed=packed, w_sum=None, scale=scale, in_features=K, out_features=N)


def random_model(cfg: BitNetConfig, seed: int = 0, norm_jitter: float = 0.0, fast: bool = False) -> PackedBitNetModel:
    """Random-init model of the given shape.  norm_jitter > 0 perturbs the norm weights away
    from 1 (tests use it so that the gamma multiply is actually exercised)."""
    rng = np.random.default_rng(seed)
    H, I = cfg.hidden_size, cfg.intermediate_size
    D = H // cfg.num_heads
    kv = cfg.num_kv_heads * D

    def gamma(n):
        g = np.ones(n, dtype=np.float32)
        if norm_jitter:
            g += rng.uniform(-norm_jitter, norm_jitter, n).astype(np.float32)
        return fp32_to_bf16_u16(g)

    layers = []
    random_projection = random_projection_fast if fast else globals()["random_projection"]
    for _ in range(cfg.num_layers):
        layers.append(PackedLayer(
            q_proj=random_projection(rng, H, H), k_proj=random_projection(rng, kv, H),
            v_proj=random_projection(rng, kv, H), o_proj=random_projection(rng, H, H),
            gate_proj=random_projection(rng, I, H), up_proj=random_projection(rng, I, H),
            down_proj=random_projection(rng, H, I),
            input_norm=gamma(H), post_attn_norm=gamma(H), attn_sub_norm=gamma(H), ffn_sub_norm=gamma(I)))
    emb = np.empty((cfg.vocab_size, H), dtype=np.uint16)
    for r in range(0, cfg.vocab_size, 8192):
        n = min(8192, cfg.vocab_size - r)
        emb[r:r + n] = fp32_to_bf16_u16(rng.standard_normal((n, H), dtype=np.float32))
    return PackedBitNetModel(config=cfg, embed_tokens=emb, final_norm=gamma(H), layers=layers)


def bitnet_2b_config(**over) -> BitNetConfig:
    d = dict(BITNET_2B)
    d.update(over)
    return BitNetConfig(**d)


def toy_config(hidden=256, layers=2, heads=4, kv_heads=2, inter=512, vocab=1024) -> BitNetConfig:
    return BitNetConfig(hidden_size=hidden, num_layers=layers, num_heads=heads, num_kv_heads=kv_heads,
                        intermediate_size=inter, vocab_size=vocab, max_position_embeddings=4096,
                        rms_norm_eps=1e-5, rope_theta=500000.0)


def random_checkpoint_tensors(cfg: BitNetConfig, seed: int = 0) -> dict:
    """Random bf16 MASTER weights of a BitNet checkpoint under their Hugging Face tensor names (uint16 bits):
    what ``loader.save_bitnet_dir`` writes and ``loader.load_bitnet_dir`` quantises."""
    rng = np.random.default_rng(seed)
    H, I = cfg.hidden_size, cfg.intermediate_size
    kv = cfg.num_kv_heads * (H // cfg.num_heads)

    def bf16(shape, std=0.02):
        return fp32_to_bf16_u16((rng.standard_normal(shape) * std).astype(np.float32))

    def gamma(n):
        return fp32_to_bf16_u16(rng.uniform(0.9, 1.1, n).astype(np.float32))

    t = {"model.embed_tokens.weight": bf16((cfg.vocab_size, H), 1.0), "model.norm.weight": gamma(H)}
    shapes = {".self_attn.q_proj.weight": (H, H), ".self_attn.k_proj.weight": (kv, H), ".self_attn.v_proj.weight": (kv, H),
              ".self_attn.o_proj.weight": (H, H), ".mlp.gate_proj.weight": (I, H), ".mlp.up_proj.weight": (I, H),
              ".mlp.down_proj.weight": (H, I)}
    norms = {".input_layernorm.weight": H, ".post_attention_layernorm.weight": H,
             ".self_attn.attn_sub_norm.weight": H, ".mlp.ffn_sub_norm.weight": I}
    for i in range(cfg.num_layers):
        for suf, shape in shapes.items():
            t[f"model.layers.{i}{suf}"] = bf16(shape)
        for suf, n in norms.items():
            t[f"model.layers.{i}{suf}"] = gamma(n)
    return t


# ---- Falcon-E family ------------------------------------------------------------------------------------------
def toy_falcon_config(hidden=256, layers=2, heads=4, kv_heads=2, inter=512, vocab=1024, eos=(2,)) -> FalconTernaryConfig:
    return FalconTernaryConfig(hidden_size=hidden, num_layers=layers, num_heads=heads, num_kv_heads=kv_heads,
                               intermediate_size=inter, vocab_size=vocab, max_position_embeddings=2048,
                               rms_norm_eps=1e-5, rope_theta=10000.0, eos_token_ids=tuple(eos))


def hf_pack_rows(t: np.ndarray) -> np.ndarray:
    """int8 {-1, 0, +1} [N, K] -> the Hugging Face BitNet packing uint8 [ceil(N / 4), K] that Falcon-E checkpoints
    store: byte (r, c) = codes of rows r, r + n, r + 2n, r + 3n at column c, two bits each (rows past N: code 1)."""
    N, K = t.shape
    n = (N + 3) // 4
    codes = np.ones((4 * n, K), dtype=np.uint8)
    codes[:N] = (t.astype(np.int16) + 1).astype(np.uint8)
    return (codes[0:n] | (codes[n:2 * n] << 2) | (codes[2 * n:3 * n] << 4) | (codes[3 * n:4 * n] << 6)).astype(np.uint8)


def random_falcon_checkpoint_tensors(cfg: FalconTernaryConfig, seed: int = 0, untied_head: bool = True) -> dict:
    """Random Falcon-E checkpoint as ``{name: (array, safetensors dtype tag)}``: ternary projections in the
    Hugging Face packing with a bf16 ``weight_scale`` (the reciprocal of the per-tensor scale), bf16 norms,
    bf16 embedding and (optionally) an untied bf16 LM head.  What ``loader.save_falcon_dir`` writes."""
    rng = np.random.default_rng(seed)
    H, I = cfg.hidden_size, cfg.intermediate_size
    kv = cfg.num_kv_heads * (H // cfg.num_heads)
    t = {"model.embed_tokens.weight": (fp32_to_bf16_u16(rng.standard_normal((cfg.vocab_size, H), dtype=np.float32)), "BF16"),
         "model.norm.weight": (fp32_to_bf16_u16(rng.uniform(0.9, 1.1, H).astype(np.float32)), "BF16")}
    if untied_head:
        t["lm_head.weight"] = (fp32_to_bf16_u16(rng.standard_normal((cfg.vocab_size, H), dtype=np.float32)), "BF16")
    shapes = {".self_attn.q_proj.weight": (H, H), ".self_attn.k_proj.weight": (kv, H), ".self_attn.v_proj.weight": (kv, H),
              ".self_attn.o_proj.weight": (H, H), ".mlp.gate_proj.weight": (I, H), ".mlp.up_proj.weight": (I, H),
              ".mlp.down_proj.weight": (H, I)}
    for i in range(cfg.num_layers):
        for suf, (N, K) in shapes.items():
            w = rng.integers(-1, 2, size=(N, K), dtype=np.int8)
            t[f"model.layers.{i}{suf}"] = (hf_pack_rows(w), "U8")
            # stored scale = 1 / w_scale, kept exactly representable in bf16
            inv = fp32_to_bf16_u16(np.array([rng.uniform(0.7, 2.0)], dtype=np.float32))
            t[f"model.layers.{i}{suf}_scale"] = (inv, "BF16")
        for suf in (".input_layernorm.weight", ".post_attention_layernorm.weight"):
            t[f"model.layers.{i}{suf}"] = (fp32_to_bf16_u16(rng.uniform(0.9, 1.1, H).astype(np.float32)), "BF16")
    return t


def random_falcon_model(cfg: FalconTernaryConfig, seed: int = 0, norm_jitter: float = 0.1) -> PackedFalconModel:
    """Random-init Falcon-E-shaped host model (SiLU gate, no sub-norms, untied bf16 LM head)."""
    rng = np.random.default_rng(seed)
    H, I = cfg.hidden_size, cfg.intermediate_size
    kv = cfg.num_kv_heads * (H // cfg.num_heads)

    def gamma(n):
        return fp32_to_bf16_u16((np.ones(n) + rng.uniform(-norm_jitter, norm_jitter, n)).astype(np.float32))

    layers = [PackedFalconLayer(
        q_proj=random_projection(rng, H, H), k_proj=random_projection(rng, kv, H), v_proj=random_projection(rng, kv, H),
        o_proj=random_projection(rng, H, H), gate_proj=random_projection(rng, I, H), up_proj=random_projection(rng, I, H),
        down_proj=random_projection(rng, H, I), input_norm=gamma(H), post_attn_norm=gamma(H))
        for _ in range(cfg.num_layers)]
    emb = fp32_to_bf16_u16(rng.standard_normal((cfg.vocab_size, H), dtype=np.float32))
    head = fp32_to_bf16_u16(rng.standard_normal((cfg.vocab_size, H), dtype=np.float32))
    return PackedFalconModel(config=cfg, embed_tokens=emb, final_norm=gamma(H), layers=layers, lm_head_tokens=head)
