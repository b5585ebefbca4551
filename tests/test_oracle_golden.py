"""The CPU oracle against outputs of the reference itself (tests/golden/*.npz, produced by
tests/golden/make_golden.py from the reference's own compiled kernels and Python runtime).

The C restatement must match the AVX-512 build bit for bit on every kernel; the AVX2 build
rounds and reduces differently in places, so it is compared exactly on integer work and within
a stated tolerance on fp32 reductions."""
import importlib

import numpy as np
import pytest

from tests.golden.make_golden import KERNEL_CASES, LM_CASES, ROW_CASES

synthetic = importlib.import_module("litespark_inference_b200.torchless.synthetic")


@pytest.fixture(scope="module")
def g512(golden_dir):
    return np.load(golden_dir / "kernels_avx512.npz")


@pytest.fixture(scope="module")
def g2(golden_dir):
    return np.load(golden_dir / "kernels_avx2.npz")


@pytest.mark.parametrize("ci", range(len(KERNEL_CASES)))
def test_matmul_bit_exact(port, g512, g2, ci):
    packed, xq, xs = g512[f"mm{ci}_packed"], g512[f"mm{ci}_xq"], g512[f"mm{ci}_xs"]
    ws = float(g512[f"mm{ci}_wscale"])
    acc = port.acc_int32(xq, packed)
    assert np.array_equal(acc, g512[f"mm{ci}_acc"])
    assert np.array_equal(acc, g2[f"mm{ci}_acc"])            # integer work: both builds agree
    y = port.matmul_packed_mT(xq, xs, packed, ws)
    assert np.array_equal(y, g512[f"mm{ci}_y"])
    y1 = np.stack([port.matmul_packed_m1(np.ascontiguousarray(xq[t]), packed, ws, float(xs[t]))
                   for t in range(xq.shape[0])])
    assert np.array_equal(y1, g512[f"mm{ci}_y"])


@pytest.mark.parametrize("ci", range(len(ROW_CASES)))
def test_row_helpers_bit_exact(port, g512, ci):
    g = {k.split("_", 1)[1]: g512[k] for k in g512.files if k.startswith(f"row{ci}_")}
    x, T, K = g["x"], *g["x"].shape
    xq, xs = np.empty((T, K), np.int8), np.empty(T, np.float32)
    port.quantize_activation_batched(x, xq, xs)
    assert np.array_equal(xq, g["xq"]) and np.array_equal(xs, g["xs"])
    out = np.empty((T, K), np.float32)
    assert np.array_equal(port.rmsnorm_into_batched(x, g["g16"], out), g["n16"])
    assert np.array_equal(port.rmsnorm_into_batched(x, g["g32"], out), g["n32"])
    rq, rs = np.empty((T, K), np.int8), np.empty(T, np.float32)
    port.rmsnorm_quantize_batched(x, g["g16"], rq, rs, np.empty((T, K), np.float32))
    assert np.array_equal(rq, g["rq"]) and np.array_equal(rs, g["rs"])
    assert np.array_equal(port.relu2_mul_into_batched(x, g["up"], out), g["r2"])
    a = x[0].copy()
    assert np.array_equal(port.add_inplace(a, np.ascontiguousarray(g["up"][0])), g["add"])


@pytest.mark.parametrize("ci", range(len(LM_CASES)))
def test_lm_head_bit_exact(port, g512, g2, ci):
    g = {k.split("_", 1)[1]: g512[k] for k in g512.files if k.startswith(f"lm{ci}_")}
    V, H = g["e16"].shape
    l16 = port.lm_head_bf16(g["e16"], g["x"], np.empty(V, np.float32))
    l8 = port.lm_head_int8(g["e8"], g["sc"], g["x"], np.empty(V, np.float32))
    l4 = port.lm_head_int4(g["e4"], g["sc"], g["x"], np.empty(V, np.float32), H)
    assert np.array_equal(l16, g["l16"])
    assert np.array_equal(l8, g["l8"])
    assert np.array_equal(l4, g["l4"])
    # the AVX2 build sums in another order: same values to fp32 reduction tolerance
    tol = 1e-5 * np.abs(g["x"]).sum() * 8
    assert np.allclose(l16, g2[f"lm{ci}_l16"], rtol=1e-4, atol=tol)
    assert np.allclose(l8, g2[f"lm{ci}_l8"], rtol=1e-4, atol=tol)
    assert np.allclose(l4, g2[f"lm{ci}_l4"], rtol=1e-4, atol=tol)


def test_host_formats(oracle, golden_dir, tl):
    g = np.load(golden_dir / "host_formats.npz")
    for impl_pack, impl_unpack in ((oracle.pack_ternary, oracle.unpack_ternary),
                                   (tl.pack.pack_ternary_4_per_byte, tl.pack.unpack_4_per_byte)):
        assert np.array_equal(impl_pack(g["pack_w"]), g["pack_packed"])
        assert np.array_equal(impl_unpack(g["pack_packed"], g["pack_w"].shape[1]), g["pack_w"])
    for impl in (oracle.quantize_ternary_absmean, tl.quantize.quantize_ternary_absmean):
        t, s = impl(g["q_in"], row_block=16)
        assert np.array_equal(t, g["q_ternary"]) and s == float(g["q_scale"])
    for impl in (oracle.rope_tables, tl.ops.rope_tables):
        c, s = impl(128, 300, 500000.0)
        assert np.array_equal(c, g["rope_cos128"]) and np.array_equal(s, g["rope_sin128"])
        c, s = impl(64, 40, 500000.0)
        assert np.array_equal(c, g["rope_cos64"]) and np.array_equal(s, g["rope_sin64"])


def _toy():
    cfg = synthetic.toy_config()
    return cfg, synthetic.random_model(cfg, seed=11, norm_jitter=0.1)


def test_runtime_restatement_matches_reference_runtime(oracle, port, golden_dir):
    """oracle.forward_* / generate* against the reference's runtime.py on the toy model."""
    g = np.load(golden_dir / "runtime_toy_avx512.npz")
    cfg, m = _toy()
    prompt = [int(t) for t in g["prompt"]]
    st = oracle.State(cfg, 64)
    step = np.stack([oracle.forward_one(port, m, st, t) for t in prompt])
    # kernels are bit-identical; attention goes through the same numpy calls -> exact here
    assert np.allclose(step, g["logits_stepwise"], rtol=1e-5, atol=1e-5)
    st = oracle.State(cfg, 64)
    lp = oracle.forward_prefill(port, m, st, prompt)
    assert np.allclose(lp, g["logits_prefill"], rtol=1e-5, atol=1e-5)
    assert oracle.generate(port, m, prompt, 24) == [int(t) for t in g["greedy24"]]
    assert oracle.generate(port, m, prompt, 24, kv_dtype=np.float16) == [int(t) for t in g["greedy24_kv16"]]
    rep = [int(t) for t in g["spec_prompt"]]
    assert oracle.generate_speculative(port, m, rep, 24, spec_k=4, match_n=4) == [int(t) for t in g["spec24"]]
    assert oracle.generate(port, m, rep, 24) == [int(t) for t in g["greedy_rep24"]]
    st = oracle.State(cfg, 64)
    oracle.forward_prefill(port, m, st, prompt[:10])
    al = oracle.forward_prefill_all_logits(port, m, st, prompt[10:15])
    assert np.allclose(al, g["all_logits"], rtol=1e-5, atol=1e-5)


def test_compiled_reference_agrees_with_port(oracle, port):
    """Where the compiled reference object can run on this CPU, drive it beside the port on
    fresh random inputs at a BitNet-2B shape (int32 exact, fp32 bit-identical for avx512)."""
    tier = oracle.ref_tier()
    if tier is None:
        pytest.skip("no compiled reference object usable on this CPU")
    ref = oracle.Kernels("ref", tier)
    rng = np.random.default_rng(5)
    N, K, T = 640, 2560, 70                 # T > 64 exercises the chunked drive of the reference
    w = rng.integers(-1, 2, (N, K), dtype=np.int8)
    packed = oracle.pack_ternary(w)
    x = rng.standard_normal((T, K)).astype(np.float32)
    xq_p, xs_p = np.empty((T, K), np.int8), np.empty(T, np.float32)
    xq_r, xs_r = np.empty((T, K), np.int8), np.empty(T, np.float32)
    port.quantize_activation_batched(x, xq_p, xs_p)
    ref.quantize_activation_batched(x, xq_r, xs_r)
    assert np.array_equal(xq_p, xq_r) and np.array_equal(xs_p, xs_r)
    assert np.array_equal(port.acc_int32(xq_p, packed), ref.acc_int32(xq_r, packed))
    assert np.array_equal(port.acc_int32(xq_p, packed), (w.astype(np.int32) @ xq_p.astype(np.int32).T).T)
    yp = port.matmul_packed_mT(xq_p, xs_p, packed, 0.8125)
    yr = ref.matmul_packed_mT(xq_r, xs_r, packed, 0.8125)
    assert np.array_equal(yp, yr)


def test_falcon_restatement_matches_reference_runtime(oracle, port, golden_dir):
    """The Falcon-E branch of the oracle (no sub-norms, SiLU gate, untied head, EOS stop) against the
    reference's falcon_forward_one / falcon_generate on the toy Falcon model."""
    g = np.load(golden_dir / "falcon_toy_avx512.npz")
    cfg = synthetic.toy_falcon_config()
    m = synthetic.random_falcon_model(cfg, seed=41)
    prompt = [int(t) for t in g["prompt"]]
    st = oracle.State(cfg, 64)
    step = np.stack([oracle.forward_one(port, m, st, t) for t in prompt])
    assert np.allclose(step, g["logits_stepwise"], rtol=1e-5, atol=1e-5)
    assert oracle.falcon_generate(port, m, prompt, 24) == [int(t) for t in g["greedy24"]]
    import copy
    m2 = copy.copy(m)
    m2.config = synthetic.toy_falcon_config(eos=(int(g["eos_id"]),))
    stopped = oracle.falcon_generate(port, m2, prompt, 24)
    assert stopped == [int(t) for t in g["greedy_until_eos"]] and len(stopped) == 3
