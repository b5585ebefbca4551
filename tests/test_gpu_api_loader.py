"""Checkpoint pipeline and facade on the device: the GPU's ternarise + pack + re-tile of bf16 master
weights against the host quantiser (the reference's, quantize.py:24-60 + pack.py:16-45), and the BitNet
facade against the runtime it wraps."""
import importlib

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

loader = importlib.import_module("litespark_inference_b200.torchless.loader")
quantize = importlib.import_module("litespark_inference_b200.torchless.quantize")
pack = importlib.import_module("litespark_inference_b200.torchless.pack")
rt = importlib.import_module("litespark_inference_b200.torchless.runtime")
api = importlib.import_module("litespark_inference_b200.torchless.api")
tk = importlib.import_module("litespark_inference_b200.torchless.tokenizer")
K = importlib.import_module("litespark_inference_b200.torchless.kernel")

synthetic = importlib.import_module("litespark_inference_b200.torchless.synthetic")


def toy_checkpoint(tmp_path, seed=3):
    cfg = synthetic.toy_config()
    t = synthetic.random_checkpoint_tensors(cfg, seed)
    loader.save_bitnet_dir(tmp_path, cfg, t)
    return cfg, t


@pytest.mark.parametrize("N,Kd,std", [(16, 64, 0.02), (33, 260, 1.0), (640, 2560, 0.02), (5, 20, 3.0), (1, 4, 0.5)])
def test_device_ternarise_equals_host_quantiser(N, Kd, std):
    rng = np.random.default_rng(N * 7 + Kd)
    w32 = (rng.standard_normal((N, Kd)) * std).astype(np.float32)
    w32[rng.random((N, Kd)) < 0.05] = 0.0
    w = quantize.fp32_to_bf16_u16(w32)
    tern, scale = quantize.quantize_ternary_absmean(w)
    lib = K.load_library(True)
    h = lib.lspk_upload_bf16_ternary(w.ctypes.data, N, Kd, float(scale))
    assert h, K.last_error()
    out = np.empty((N, Kd // 4), np.uint8)
    K.check(lib.lspk_download_packed(h, out))
    import ctypes
    sc = ctypes.c_float(0)
    K.check(lib.lspk_weight_shape(h, None, None, ctypes.byref(sc), None))
    lib.lspk_weight_free(h)
    assert np.array_equal(out, pack.pack_ternary_4_per_byte(tern))
    assert sc.value == np.float32(scale)


def test_loader_device_path_equals_host_path(tmp_path):
    cfg, _ = toy_checkpoint(tmp_path)
    host = loader.load_bitnet_dir(tmp_path, embed_dtype="bf16", device_quantize=False)
    devm = loader.load_bitnet_dir(tmp_path, embed_dtype="bf16", device_quantize=True)
    assert all(getattr(L, k).w_packed is None and getattr(L, k).w_bf16 is None for L in devm.layers for k in loader._PROJ_SUFFIX)
    prompt = [int(t) for t in np.random.default_rng(4).integers(0, cfg.vocab_size, 21)]
    a = rt.generate(rt.to_device(host), prompt, 16)
    b = rt.generate(rt.to_device(devm), prompt, 16)
    assert a == b
    dm = rt.to_device(devm)
    lib = dm.lib
    for li, L in enumerate(host.layers):
        for name in ("q_proj", "down_proj"):
            p = getattr(L, name)
            out = np.empty_like(p.w_packed)
            K.check(lib.lspk_download_packed(dm.projection(li, name), out))
            assert np.array_equal(out, p.w_packed)


def test_facade_generate_matches_runtime(tmp_path):
    cfg, _ = toy_checkpoint(tmp_path)
    model = loader.load_bitnet_dir(tmp_path, embed_dtype="int4", device_quantize=True)
    bn = api.BitNet(model, tk.IdTokenizer(), default_t_max=64)
    prompt = [int(t) for t in np.random.default_rng(6).integers(0, cfg.vocab_size, 12)]
    want = rt.generate(rt.to_device(model), prompt, 20)
    text = bn.generate(" ".join(map(str, prompt)), 20)
    assert [int(t) for t in text.split()] == want
    full = bn.generate(prompt, 20, return_full=True)
    assert full.token_ids == want and full.prompt_tokens == 12 and full.generated_tokens == 20
    assert full.gen_tok_per_s > 0 and full.prefill_tok_per_s > 0 and not full.speculative
    # speculative decoding returns the greedy tokens (repetitive prompt so that the lookup proposes something)
    rep = (prompt[:4] * 6)[:22]
    spec = bn.generate(rep, 20, speculative=True, return_full=True)
    assert spec.token_ids == rt.generate(rt.to_device(model), rep, 20) and spec.speculative and spec.spec_stats
    paths = bn.kernel_paths()
    assert paths["extension"].endswith("_lspk_sm100.so") and paths["has_batched_matmul"] and not paths["has_amx"]
    mem = bn.memory_bytes()
    assert mem["device_bytes"] > 0
    bench = bn.benchmark([prompt], max_new_tokens=4, runs=2)
    assert bench["summary"]["median_gen_tok_per_s"] > 0 and len(bench["results"][0]["gen_tok_per_s"]) == 2
    with pytest.raises(ValueError):
        bn.generate([], 4)
