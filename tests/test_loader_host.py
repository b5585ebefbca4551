"""Host side of the checkpoint pipeline: safetensors container, embedding quantisers against the
reference loader's outputs (golden fixtures), and the host path of the loader on a synthetic checkpoint."""
import importlib
import struct

import numpy as np
import pytest

loader = importlib.import_module("litespark_inference_b200.torchless.loader")
sio = importlib.import_module("litespark_inference_b200.torchless.safetensors_io")
quantize = importlib.import_module("litespark_inference_b200.torchless.quantize")
pack = importlib.import_module("litespark_inference_b200.torchless.pack")
synthetic = importlib.import_module("litespark_inference_b200.torchless.synthetic")


def toy_checkpoint(tmp_path, seed=3):
    """Random bf16 master weights of the toy shape, written as a checkpoint directory."""
    cfg = synthetic.toy_config()
    t = synthetic.random_checkpoint_tensors(cfg, seed)
    loader.save_bitnet_dir(tmp_path, cfg, t)
    return cfg, t


def test_safetensors_round_trip_and_validation(tmp_path):
    rng = np.random.default_rng(0)
    a = rng.standard_normal((5, 7)).astype(np.float32)
    b = rng.integers(0, 65535, (3, 4, 2)).astype(np.uint16)
    c = np.zeros((0, 4), np.int8)                                   # empty tensor
    p = tmp_path / "x.safetensors"
    sio.save_safetensors(p, {"a": (a, "F32"), "b": (b, "BF16"), "c": (c, "I8")})
    sf = sio.open_safetensors(p)
    assert set(sf.keys()) == {"a", "b", "c"} and "a" in sf and "zz" not in sf
    va, ta = sf.view("a")
    gb, tb = sf.get("b")
    assert ta == "F32" and tb == "BF16" and np.array_equal(va, a) and np.array_equal(gb, b)
    assert sf.get("c")[0].shape == (0, 4)
    with pytest.raises(KeyError):
        sf.view("missing")
    # truncated data section and a header that lies about a shape are rejected
    raw = p.read_bytes()
    (tmp_path / "short.safetensors").write_bytes(raw[:-8])
    with pytest.raises(ValueError):
        sio.open_safetensors(tmp_path / "short.safetensors")
    (n,) = struct.unpack("<Q", raw[:8])
    bad = raw[:8] + raw[8:8 + n].replace(b'"shape":[5,7]', b'"shape":[5,8]') + raw[8 + n:]
    (tmp_path / "bad.safetensors").write_bytes(bad)
    with pytest.raises(ValueError):
        sio.open_safetensors(tmp_path / "bad.safetensors")
    (tmp_path / "tiny.safetensors").write_bytes(b"abc")
    with pytest.raises(ValueError):
        sio.open_safetensors(tmp_path / "tiny.safetensors")


def test_embedding_quantisers_match_reference_loader(golden_dir):
    g = np.load(golden_dir / "host_formats.npz")
    q8, s8 = loader.quantize_embedding(g["emb_in"], 127, row_block=32)
    q4, s4 = loader.quantize_embedding(g["emb_in"], 7, row_block=32)
    assert np.array_equal(q8, g["emb_int8"]) and np.array_equal(s8, g["emb_int8_scale"])
    assert np.array_equal(q4, g["emb_int4"]) and np.array_equal(s4, g["emb_int4_scale"])
    with pytest.raises(ValueError):
        loader.quantize_embedding(np.zeros((2, 3), np.uint16), 7)


@pytest.mark.parametrize("embed_dtype", ["bf16", "int8", "int4"])
def test_loader_host_path(tmp_path, embed_dtype):
    cfg, t = toy_checkpoint(tmp_path)
    m = loader.load_bitnet_dir(tmp_path, embed_dtype=embed_dtype, device_quantize=False)
    assert m.config == cfg and len(m.layers) == cfg.num_layers
    for i, L in enumerate(m.layers):
        for k, suf in loader._PROJ_SUFFIX.items():
            w = t[f"model.layers.{i}{suf}"]
            tern, scale = quantize.quantize_ternary_absmean(w)
            p = getattr(L, k)
            assert p.scale == scale and (p.out_features, p.in_features) == w.shape
            assert np.array_equal(p.w_packed, pack.pack_ternary_4_per_byte(tern))
            assert np.array_equal(p.w_sum, tern.sum(axis=1, dtype=np.int32))
        assert np.array_equal(L.ffn_sub_norm, t[f"model.layers.{i}.mlp.ffn_sub_norm.weight"])
    emb = t["model.embed_tokens.weight"]
    if embed_dtype == "bf16":
        assert np.array_equal(m.embed_tokens, emb) and m.embed_int8 is None and m.embed_int4 is None
    elif embed_dtype == "int8":
        assert m.embed_tokens is None and m.embed_int8.shape == emb.shape and m.embed_scale.shape == (cfg.vocab_size,)
    else:
        assert m.embed_int4.shape == (cfg.vocab_size, cfg.hidden_size // 2)


def test_loader_rejects_bad_input(tmp_path):
    with pytest.raises(FileNotFoundError):
        loader.load_bitnet_dir(tmp_path / "nowhere")
    toy_checkpoint(tmp_path)
    with pytest.raises(ValueError):
        loader.load_bitnet_dir(tmp_path, embed_dtype="fp8", device_quantize=False)


def test_falcon_packing_and_loader_match_reference(tmp_path, golden_dir):
    """The Hugging Face row-blocked packing of Falcon-E checkpoints against the reference loader's own outputs
    (fixture generated from its _unpack_hf_packed_bitnet / _load_falcon_proj), then a whole synthetic checkpoint
    through load_falcon_dir."""
    g = np.load(golden_dir / "falcon_toy_avx512.npz")
    assert np.array_equal(loader.unpack_hf_packed_bitnet(g["hf_packed"], 37), g["hf_unpacked"])
    assert np.array_equal(synthetic.hf_pack_rows(g["hf_unpacked"]), g["hf_packed"])
    sio.save_safetensors(tmp_path / "one.safetensors", {"w": (g["hf_packed"], "U8"),
                                                        "w_scale": (np.array([0x3FC0], np.uint16), "BF16")})
    sf = sio.open_safetensors(tmp_path / "one.safetensors")
    p = loader.load_falcon_projection(sf, "w", 37)
    assert np.array_equal(p.w_packed, g["hf_proj_packed"]) and p.scale == float(g["hf_proj_scale"])
    assert (p.out_features, p.in_features) == (37, 24)
    # whole checkpoint: shapes, scales (reciprocal of the stored tensor), untied head, EOS list
    cfg = synthetic.toy_falcon_config(eos=(2, 7))
    t = synthetic.random_falcon_checkpoint_tensors(cfg, seed=4)
    loader.save_falcon_dir(tmp_path / "ckpt", cfg, t)
    for embed_dtype in ("bf16", "int8", "int4"):
        m = loader.load_falcon_dir(tmp_path / "ckpt", embed_dtype=embed_dtype)
        assert m.config == cfg and len(m.layers) == cfg.num_layers
        L = m.layers[1]
        raw, _ = t["model.layers.1.mlp.down_proj.weight"]
        assert np.array_equal(pack.unpack_4_per_byte(L.down_proj.w_packed, cfg.intermediate_size),
                              loader.unpack_hf_packed_bitnet(raw, cfg.hidden_size))
        inv = quantize.bf16_u16_to_fp32(t["model.layers.1.mlp.down_proj.weight_scale"][0])[0]
        assert L.down_proj.scale == float(1.0 / inv)
        assert L.attn_sub_norm is None and L.ffn_sub_norm is None
        tables = {"bf16": (m.embed_tokens, m.lm_head_tokens), "int8": (m.embed_int8, m.lm_head_int8),
                  "int4": (m.embed_int4, m.lm_head_int4)}[embed_dtype]
        assert tables[0] is not None and tables[1] is not None and not np.array_equal(tables[0], tables[1])
    # a checkpoint without lm_head.weight ties the head to the embedding
    t2 = {k: v for k, v in t.items() if k != "lm_head.weight"}
    loader.save_falcon_dir(tmp_path / "tied", cfg, t2)
    m = loader.load_falcon_dir(tmp_path / "tied", embed_dtype="bf16")
    assert m.lm_head_tokens is m.embed_tokens
    with pytest.raises(FileNotFoundError):
        loader.load_falcon_dir(tmp_path / "nowhere")
