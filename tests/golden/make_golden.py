"""Generate the golden fixtures in this directory from the REFERENCE itself.

Run where the reference tree is present (its location: environment variable LSPK_REFERENCE_ROOT) with its compiled
kernels under oracle/_ref (``make -C oracle ref``):

    python tests/golden/make_golden.py

It imports the reference's own Python package (``litespark_inference.torchless``: pack,
quantize, ops, kernel, runtime) with its ctypes loader pointed at the compiled reference object,
feeds it small seeded inputs and stores inputs' seeds plus the reference's outputs as .npz.
The tests rebuild the inputs from the same seeds, so the files stay small.  Nothing here is
imported by the tests or the library.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))

import __graft_entry__ as entry  # noqa: E402

entry.load_package()
from litespark_inference_b200.torchless import synthetic  # noqa: E402


def reference_modules(tier: str):
    """Import the reference's torchless modules, bound to oracle/_ref/_matmul_lut_<tier>.so."""
    if not os.environ.get("LSPK_REFERENCE_ROOT"):
        sys.exit("set LSPK_REFERENCE_ROOT to a checkout of the reference (its Python package is imported from there)")
    ref = str(Path(os.environ["LSPK_REFERENCE_ROOT"]))
    if ref not in sys.path:
        sys.path.insert(0, ref)
    os.environ["LITESPARK_KERNEL_TIER"] = tier
    for m in [m for m in sys.modules if m.startswith("litespark_inference.")]:
        del sys.modules[m]
    import importlib
    kernel = importlib.import_module("litespark_inference.torchless.kernel")
    so = ROOT / "oracle" / "_ref" / f"_matmul_lut_{tier}.so"
    kernel._find_built_extension = lambda: so       # the tree is read-only: no in-place build
    kernel._lib = None
    kernel._load()
    runtime = importlib.import_module("litespark_inference.torchless.runtime")
    pack = importlib.import_module("litespark_inference.torchless.pack")
    quantize = importlib.import_module("litespark_inference.torchless.quantize")
    ops = importlib.import_module("litespark_inference.torchless.ops")
    model = importlib.import_module("litespark_inference.torchless.model")
    return kernel, runtime, pack, quantize, ops, model


def to_reference_model(refmodel, m):
    """Rebuild a synthetic model with the reference's own container classes."""
    c = m.config
    cfg = refmodel.BitNetConfig(c.hidden_size, c.num_layers, c.num_heads, c.num_kv_heads, c.intermediate_size,
                                c.vocab_size, c.max_position_embeddings, c.rms_norm_eps, c.rope_theta)

    def proj(p):
        return refmodel.PackedProjection(w_packed=p.w_packed, w_sum=np.zeros(p.out_features, np.int32),
                                         scale=p.scale, in_features=p.in_features, out_features=p.out_features)
    layers = [refmodel.PackedLayer(proj(L.q_proj), proj(L.k_proj), proj(L.v_proj), proj(L.o_proj),
                                   proj(L.gate_proj), proj(L.up_proj), proj(L.down_proj),
                                   L.input_norm, L.post_attn_norm, L.attn_sub_norm, L.ffn_sub_norm)
              for L in m.layers]
    return refmodel.PackedBitNetModel(config=cfg, embed_tokens=m.embed_tokens, final_norm=m.final_norm,
                                      layers=layers, embed_int8=m.embed_int8, embed_scale=m.embed_scale,
                                      embed_int4=m.embed_int4)


KERNEL_CASES = [  # (N, K, T): ragged sizes exercise the scalar tails of the reference kernels
    (48, 128, 1), (5, 20, 1), (33, 260, 3), (64, 1024, 8), (17, 64, 64), (130, 448, 5),
]
ROW_CASES = [(1, 64), (3, 100), (2, 2560), (1, 6912), (4, 37)]
LM_CASES = [(70, 64), (257, 96), (64, 2560)]


def gen_kernels(tier: str):
    kernel, runtime, pack, quantize, ops, model = reference_modules(tier)
    out = {}
    for ci, (N, K, T) in enumerate(KERNEL_CASES):
        rng = np.random.default_rng(1000 + ci)
        w = rng.integers(-1, 2, (N, K), dtype=np.int8)
        packed = pack.pack_ternary_4_per_byte(w)
        x = (rng.standard_normal((T, K)) * rng.uniform(0.1, 4.0)).astype(np.float32)
        xq = np.empty((T, K), np.int8)
        xs = np.empty(T, np.float32)
        for t in range(T):
            xs[t] = kernel.quantize_activation(np.ascontiguousarray(x[t]), xq[t])
        w_scale = float(np.float32(rng.uniform(0.5, 1.5)))
        y1 = np.stack([kernel.matmul_packed_m1(np.ascontiguousarray(xq[t]), packed, w_scale, float(xs[t]))
                       for t in range(T)])
        yT = kernel.matmul_packed_mT(xq, xs, packed, w_scale)
        acc = kernel.matmul_packed_mT(xq, np.ones(T, np.float32), packed, 1.0)
        assert np.array_equal(y1, yT)
        out[f"mm{ci}_packed"] = packed
        out[f"mm{ci}_xq"] = xq
        out[f"mm{ci}_xs"] = xs
        out[f"mm{ci}_wscale"] = np.float32(w_scale)
        out[f"mm{ci}_y"] = yT
        out[f"mm{ci}_acc"] = acc.astype(np.int32)
        assert np.array_equal(acc.astype(np.int32).astype(np.float32), acc)
        assert np.array_equal(pack.unpack_4_per_byte(packed, K), w)
    for ci, (T, K) in enumerate(ROW_CASES):
        rng = np.random.default_rng(2000 + ci)
        x = (rng.standard_normal((T, K)) * 3.0).astype(np.float32)
        g32 = rng.uniform(0.5, 1.5, K).astype(np.float32)
        g16 = (g32.view(np.uint32) >> 16).astype(np.uint16)
        xq = np.empty((T, K), np.int8)
        xs = np.empty(T, np.float32)
        kernel.quantize_activation_batched(x, xq, xs)
        n16 = np.empty((T, K), np.float32)
        n32 = np.empty((T, K), np.float32)
        kernel.rmsnorm_into_batched(x, g16, n16, 1e-5)
        kernel.rmsnorm_into_batched(x, g32, n32, 1e-5)
        rq = np.empty((T, K), np.int8)
        rs = np.empty(T, np.float32)
        kernel.rmsnorm_quantize_batched(x, g16, rq, rs, np.empty((T, K), np.float32), 1e-5)
        up = rng.standard_normal((T, K)).astype(np.float32)
        r2 = np.empty((T, K), np.float32)
        kernel.relu2_mul_into_batched(x, up, r2)
        a = x[0].copy()
        kernel.add_inplace(a, np.ascontiguousarray(up[0]))
        for k_, v_ in dict(x=x, g32=g32, g16=g16, xq=xq, xs=xs, n16=n16, n32=n32, rq=rq, rs=rs, up=up, r2=r2,
                           add=a).items():
            out[f"row{ci}_{k_}"] = v_
    for ci, (V, H) in enumerate(LM_CASES):
        rng = np.random.default_rng(3000 + ci)
        e32 = rng.standard_normal((V, H)).astype(np.float32)
        e16 = (e32.view(np.uint32) >> 16).astype(np.uint16)
        e8 = rng.integers(-127, 128, (V, H), dtype=np.int8)
        e4 = rng.integers(0, 256, (V, H // 2), dtype=np.uint8)
        sc = rng.uniform(0.001, 0.01, V).astype(np.float32)
        x = rng.standard_normal(H).astype(np.float32)
        l16 = kernel.lm_head_bf16(e16, x, np.empty(V, np.float32))
        l8 = kernel.lm_head_int8(e8, sc, x, np.empty(V, np.float32))
        l4 = kernel.lm_head_int4(e4, sc, x, np.empty(V, np.float32), H)
        for k_, v_ in dict(e16=e16, e8=e8, e4=e4, sc=sc, x=x, l16=l16, l8=l8, l4=l4).items():
            out[f"lm{ci}_{k_}"] = v_
    np.savez_compressed(HERE / f"kernels_{tier}.npz", **out)
    print(f"kernels_{tier}.npz: {len(out)} arrays")


def gen_host():
    kernel, runtime, pack, quantize, ops, model = reference_modules("avx512")
    out = {}
    rng = np.random.default_rng(7)
    w = rng.integers(-1, 2, (9, 37), dtype=np.int8)
    out["pack_w"] = w
    out["pack_packed"] = pack.pack_ternary_4_per_byte(w)
    wb = (rng.standard_normal((40, 48)).astype(np.float32) * 0.02)
    wb16 = (wb.view(np.uint32) >> 16).astype(np.uint16)
    t, s = quantize.quantize_ternary_absmean(wb16, row_block=16)
    out["q_in"] = wb16
    out["q_ternary"] = t
    out["q_scale"] = np.float64(s)
    # embedding quantisers of the reference's loader (loader.py:153-219) on a small bf16 table, with a row
    # block smaller than the table so that the block loop is exercised
    import importlib
    loader = importlib.import_module("litespark_inference.torchless.loader")
    e32 = rng.standard_normal((70, 48)).astype(np.float32)
    e32[5] = 0.0                                            # an all-zero row takes the 1e-5 floor
    e16 = (e32.view(np.uint32) >> 16).astype(np.uint16)
    out["emb_in"] = e16
    out["emb_int8"], out["emb_int8_scale"] = loader._quantize_embedding_int8(e16, row_block=32)
    out["emb_int4"], out["emb_int4_scale"] = loader._quantize_embedding_int4(e16, row_block=32)
    cos, sin = ops.rope_tables(128, 300, 500000.0)
    out["rope_cos128"] = cos
    out["rope_sin128"] = sin
    cos, sin = ops.rope_tables(64, 40, 500000.0)
    out["rope_cos64"] = cos
    out["rope_sin64"] = sin
    np.savez_compressed(HERE / "host_formats.npz", **out)
    print("host_formats.npz")


def gen_runtime(tier: str):
    """Toy-model forward passes through the reference's own runtime.py."""
    kernel, runtime, pack, quantize, ops, refmodel = reference_modules(tier)
    out = {}
    cfg = synthetic.toy_config()
    m = synthetic.random_model(cfg, seed=11, norm_jitter=0.1)
    rm = to_reference_model(refmodel, m)
    prompt = [int(t) for t in np.random.default_rng(12).integers(0, cfg.vocab_size, 20)]
    out["prompt"] = np.array(prompt, np.int32)
    # decode-only path: forward_one over the prompt, logits at every position
    st = runtime.init_state(rm, 64)
    out["logits_stepwise"] = np.stack([runtime.forward_one(rm, st, t).copy() for t in prompt])
    # batched prefill (T = 20 <= 64) + greedy decode
    st = runtime.init_state(rm, 64)
    out["logits_prefill"] = runtime.forward_prefill(rm, st, prompt).copy()
    out["greedy24"] = np.array(runtime.generate(rm, prompt, 24), np.int32)
    # speculative decode on a repetitive prompt, so that the lookup finds candidates
    rep = (prompt[:5] * 5)[:24]
    out["spec_prompt"] = np.array(rep, np.int32)
    toks, stats = runtime.generate_speculative(rm, rep, 24, spec_k=4, match_n=4, return_stats=True)
    out["spec24"] = np.array(toks, np.int32)
    out["greedy_rep24"] = np.array(runtime.generate(rm, rep, 24), np.int32)
    out["spec_steps"] = np.int32(stats["steps"])
    # all-position logits of a short batch (speculative validation path)
    st = runtime.init_state(rm, 64)
    runtime.forward_prefill(rm, st, prompt[:10])
    out["all_logits"] = runtime.forward_prefill_all_logits(rm, st, prompt[10:15]).copy()
    # fp16 KV cache: the reference's arrays swapped for float16 (assignment rounds, matmul widens)
    st = runtime.init_state(rm, 64)
    st.cache_k = st.cache_k.astype(np.float16)
    st.cache_v = st.cache_v.astype(np.float16)
    out["greedy24_kv16"] = np.array(runtime.generate(rm, prompt, 24, state=st), np.int32)
    np.savez_compressed(HERE / f"runtime_toy_{tier}.npz", **out)
    print(f"runtime_toy_{tier}.npz")


def gen_falcon(tier: str):
    """Falcon-E family through the reference's own runtime (falcon_forward_one / falcon_generate) and loader
    (_unpack_hf_packed_bitnet / _load_falcon_proj), on a toy model and a toy checkpoint tensor."""
    kernel, runtime, pack, quantize, ops, refmodel = reference_modules(tier)
    import importlib
    loader = importlib.import_module("litespark_inference.torchless.loader")
    out = {}
    cfg = synthetic.toy_falcon_config()
    m = synthetic.random_falcon_model(cfg, seed=41)
    rcfg = refmodel.FalconTernaryConfig(cfg.hidden_size, cfg.num_layers, cfg.num_heads, cfg.num_kv_heads,
                                        cfg.intermediate_size, cfg.vocab_size, cfg.max_position_embeddings,
                                        cfg.rms_norm_eps, cfg.rope_theta, cfg.eos_token_ids)

    def proj(p):
        return refmodel.PackedProjection(w_packed=p.w_packed, w_sum=np.zeros(p.out_features, np.int32),
                                         scale=p.scale, in_features=p.in_features, out_features=p.out_features)
    layers = [refmodel.PackedFalconLayer(proj(L.q_proj), proj(L.k_proj), proj(L.v_proj), proj(L.o_proj),
                                         proj(L.gate_proj), proj(L.up_proj), proj(L.down_proj),
                                         L.input_norm, L.post_attn_norm) for L in m.layers]
    rm = refmodel.PackedFalconModel(config=rcfg, embed_tokens=m.embed_tokens, final_norm=m.final_norm,
                                    projection_backend="neon", layers=layers, lm_head_tokens=m.lm_head_tokens)
    prompt = [int(t) for t in np.random.default_rng(42).integers(3, cfg.vocab_size, 14)]
    out["prompt"] = np.array(prompt, np.int32)
    st = runtime.init_state(rm, 64)
    out["logits_stepwise"] = np.stack([runtime.falcon_forward_one(rm, st, t).copy() for t in prompt])
    out["greedy24"] = np.array(runtime.falcon_generate(rm, prompt, 24), np.int32)
    # generation that meets an end-of-sequence id: make the first greedy token the EOS id and generate again
    eos_cfg = refmodel.FalconTernaryConfig(cfg.hidden_size, cfg.num_layers, cfg.num_heads, cfg.num_kv_heads,
                                           cfg.intermediate_size, cfg.vocab_size, cfg.max_position_embeddings,
                                           cfg.rms_norm_eps, cfg.rope_theta, (int(out["greedy24"][3]),))
    rm.config = eos_cfg
    out["eos_id"] = np.int32(out["greedy24"][3])
    out["greedy_until_eos"] = np.array(runtime.falcon_generate(rm, prompt, 24), np.int32)
    # loader: the Hugging Face row-blocked packing, ragged row count (37 rows in 10 byte rows)
    rng = np.random.default_rng(43)
    w = rng.integers(-1, 2, (37, 24), dtype=np.int8)
    hf = synthetic.hf_pack_rows(w)
    out["hf_packed"] = hf
    out["hf_unpacked"] = loader._unpack_hf_packed_bitnet(hf, 37)
    assert np.array_equal(out["hf_unpacked"], w)

    class FakeFile:                     # the two members _load_falcon_proj touches
        header = {"w": {}, "w_scale": {}}

        @staticmethod
        def get(key):
            return (hf, "U8") if key == "w" else (np.array([0x3FC0], np.uint16), "BF16")      # bf16 1.5
    p = loader._load_falcon_proj(FakeFile, "w", 37, "neon")
    out["hf_proj_packed"] = p.w_packed
    out["hf_proj_scale"] = np.float64(p.scale)
    np.savez_compressed(HERE / f"falcon_toy_{tier}.npz", **out)
    print(f"falcon_toy_{tier}.npz")


if __name__ == "__main__":
    if "--falcon-only" in sys.argv:
        gen_falcon("avx512")
        sys.exit(0)
    gen_host()
    for tier in ("avx512", "avx2"):
        gen_kernels(tier)
    gen_runtime("avx512")
    gen_falcon("avx512")
