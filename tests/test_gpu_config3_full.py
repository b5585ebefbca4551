"""The full BitNet-2B-shaped decoder (30 layers, hidden 2560, 20 / 5 heads of 128, FFN 6912, vocabulary
128256, bf16 tied embedding) on the device against the CPU oracle: a 128-token prompt followed by 128
teacher-forced decode steps, with the fp16 and with the fp32 KV cache.

What is asserted is the band that test_gpu_bitnet_shape.py explains: a random-init network of this width
amplifies a single int8 activation that rounds the other way, so the reference's own AVX-512 and AVX2
builds do not produce the same tokens either.  The device has to stay at least as close to the AVX-512
arithmetic as the AVX2 build does (median relative L2 of the logits within a factor of 1.5, greedy
agreement within 15 points: both sides are single realisations of which activations flip), and must be
exact to fp32 rounding where nothing can have flipped yet.  The numbers behind the assertions are
printed (run with -s): per-step error quantiles, greedy agreement, top-1 / top-2 margins of the oracle's
logits at the steps where the device's choice differs, and -- from a layer-by-layer walk of the first
token through lspk_linear with its int8 tap -- the first layer and stage at which a quantised activation
differs from the oracle's.
"""
import ctypes
import importlib

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

K = importlib.import_module("litespark_inference_b200.torchless.kernel")
rt = importlib.import_module("litespark_inference_b200.torchless.runtime")
synthetic = importlib.import_module("litespark_inference_b200.torchless.synthetic")

PROMPT, STEPS = 128, 128
MEDIAN_REL_L2_NO_REF = 0.5    # absolute fallback where the compiled reference kernels cannot run


@pytest.fixture(scope="module")
def full():
    cfg = synthetic.bitnet_2b_config()
    m = synthetic.random_model(cfg, seed=17, norm_jitter=0.1, fast=True)
    dm = rt.to_device(m)
    yield cfg, m, dm
    dm.close()


def _rel_l2(got, want):
    return float(np.linalg.norm(got - want) / np.linalg.norm(want - want.mean()))


def _margin(logits):
    """(top-1 - top-2) / spread of one logits row."""
    top2 = np.partition(logits, -2)[-2:]
    return float((top2[1] - top2[0]) / (logits.max() - logits.min()))


def _ref_kernels(oracle):
    try:
        return oracle.Kernels("ref", "avx512"), oracle.Kernels("ref", "avx2")
    except (RuntimeError, OSError):
        return None, None


@pytest.mark.parametrize("kv", ["fp16", "fp32"])
def test_pp128_tg128_teacher_forced_band(full, oracle, port, kv):
    cfg, m, dm = full
    np_kv = np.float32 if kv == "fp32" else np.float16
    prompt = [int(t) for t in np.random.default_rng(4).integers(0, cfg.vocab_size, PROMPT)]
    k512, k2 = _ref_kernels(oracle)
    toks, want = oracle.generate(k512 or port, m, prompt, STEPS, kv_dtype=np_kv, return_logits=True)
    toks = [int(t) for t in toks]

    st = rt.init_state(dm, PROMPT + STEPS + 1, kv_dtype=kv)
    got = [rt.forward_prefill(dm, st, prompt)]
    for t in toks[:-1]:
        got.append(rt.forward_one(dm, st, t))
    assert st.pos == PROMPT + STEPS - 1
    st.close()

    errs = np.array([_rel_l2(g, w) for g, w in zip(got, want)])
    picks = [int(np.argmax(g)) for g in got]
    agree = float(np.mean([p == t for p, t in zip(picks, toks)]))
    margins = np.array([_margin(w) for w in want])
    miss = [i for i, (p, t) in enumerate(zip(picks, toks)) if p != t]
    print(f"\n[config 3, {kv} KV] device vs AVX-512 arithmetic over {STEPS} teacher-forced steps after pp{PROMPT}: "
          f"rel-L2 of logits min {errs.min():.3e} median {np.median(errs):.3e} max {errs.max():.3e}; "
          f"greedy agreement {agree:.3f}; oracle top-1/top-2 margin (fraction of the logit spread) "
          f"min {margins.min():.2e} median {np.median(margins):.2e}; "
          f"at the {len(miss)} steps where the device chooses differently: median margin "
          f"{(np.median(margins[miss]) if miss else float('nan')):.2e}")
    if k2 is None:
        assert float(np.median(errs)) <= MEDIAN_REL_L2_NO_REF
        return
    st2 = oracle.State(cfg, PROMPT + STEPS + 1, np_kv)
    other = [oracle.forward_prefill(k2, m, st2, prompt)]
    for t in toks[:-1]:
        other.append(oracle.forward_one(k2, m, st2, t))
    band = np.array([_rel_l2(o, w) for o, w in zip(other, want)])
    agree2 = float(np.mean([int(np.argmax(o)) == t for o, t in zip(other, toks)]))
    print(f"[config 3, {kv} KV] the reference's AVX2 build vs its AVX-512 build on the same steps: rel-L2 median "
          f"{np.median(band):.3e} max {band.max():.3e}; greedy agreement {agree2:.3f}")
    # medians of single realisations of a chaotic process on both sides: same order of magnitude, not last digit
    assert float(np.median(errs)) <= 1.5 * float(np.median(band)) + 1e-3
    assert agree >= agree2 - 0.15


def _dev(lib, a):
    p = lib.lspk_malloc(a.nbytes)
    assert p
    K.check(lib.lspk_h2d(p, a.ctypes.data_as(ctypes.c_void_p), a.nbytes))
    return p


def _host(lib, p, shape, dtype):
    out = np.empty(shape, dtype)
    K.check(lib.lspk_d2h(out.ctypes.data_as(ctypes.c_void_p), p, out.nbytes))
    return out


def _layer_walk(full, oracle, port, resync):
    """Position 0 through all 30 layers, stage by stage, through lspk_linear with the quantised-activation tap,
    beside the oracle doing the same: attention over a single key is the value row itself, so the walk needs no
    attention kernel.  resync: after every stage the device buffers are overwritten with the oracle's values, so
    that each stage is judged on identical input.  Returns per-stage records (layer, stage, differing int8
    activations, their largest difference, relative L2 of the stage's fp32 output) and the final hidden error."""
    cfg, m, dm = full
    lib = dm.lib
    H, I = cfg.hidden_size, cfg.intermediate_size
    Q, KV = cfg.num_heads, cfg.num_kv_heads
    D = H // Q
    kvd = KV * D
    eps = cfg.rms_norm_eps
    x = oracle.embed_row(m, 4242)
    d_x = _dev(lib, x)
    d_q, d_k, d_v = (lib.lspk_malloc(n * 4) for n in (H, kvd, kvd))
    d_attn, d_inter = lib.lspk_malloc(H * 4), lib.lspk_malloc(I * 4)
    d_xq, d_xs = lib.lspk_malloc(I), lib.lspk_malloc(16)
    gammas = {}

    def gamma_dev(g):
        key = g.ctypes.data
        if key not in gammas:
            gammas[key] = _dev(lib, np.ascontiguousarray(g))
        return gammas[key]

    def put(p, a):
        a = np.ascontiguousarray(a, dtype=np.float32)
        K.check(lib.lspk_h2d(p, a.ctypes.data_as(ctypes.c_void_p), a.nbytes))

    def linear(names, li, outs, src, gamma, Kdim, epilogue):
        a = K.LinearArgs()
        for i, nme in enumerate(names):
            a.w[i] = dm.projection(li, nme)
            a.out[i] = outs[i]
        a.n_mats, a.M = len(names), 1
        a.prologue, a.epilogue = K.PRO_RMSNORM_QUANT, epilogue
        a.x_f32, a.gamma, a.gamma_is_bf16, a.eps = src, gamma_dev(gamma), 1, eps
        a.xq_out, a.xscale_out = d_xq, d_xs
        K.check(lib.lspk_linear(ctypes.byref(a)))
        return _host(lib, d_xq, Kdim, np.int8)

    def oracle_q(v, gamma):
        q8, tmp = np.empty(v.shape[0], np.int8), np.empty(v.shape[0], np.float32)
        return q8, port.rmsnorm_quantize_into(np.ascontiguousarray(v), gamma, q8, tmp, eps)

    ox = x.copy()
    records = []
    for li, L in enumerate(m.layers):
        for stage in ("qkv", "o", "gate_up", "down"):
            if stage == "qkv":
                dq = linear(("q_proj", "k_proj", "v_proj"), li, (d_q, d_k, d_v), d_x, L.input_norm, H, K.EPI_STORE)
                oq, osc = oracle_q(ox, L.input_norm)
                ov = port.matmul_packed_m1(oq, L.v_proj.w_packed, np.float32(L.v_proj.scale), osc)
                v = _host(lib, d_v, kvd, np.float32)
                got, want = v, ov
                # one key: softmax weight 1, every query head of a group receives its group's value row
                o_attn = np.repeat(ov.reshape(KV, D), Q // KV, axis=0).reshape(-1)
                put(d_attn, o_attn if resync else np.repeat(v.reshape(KV, D), Q // KV, axis=0).reshape(-1))
            elif stage == "o":
                dq = linear(("o_proj",), li, (d_x,), d_attn, L.attn_sub_norm, H, K.EPI_ADD)
                oq, osc = oracle_q(o_attn, L.attn_sub_norm)
                ox = ox + port.matmul_packed_m1(oq, L.o_proj.w_packed, np.float32(L.o_proj.scale), osc)
                got, want = _host(lib, d_x, H, np.float32), ox
                if resync:
                    put(d_x, ox)
            elif stage == "gate_up":
                dq = linear(("gate_proj", "up_proj"), li, (d_inter, None), d_x, L.post_attn_norm, H, K.EPI_RELU2_MUL)
                oq, osc = oracle_q(ox, L.post_attn_norm)
                g = port.matmul_packed_m1(oq, L.gate_proj.w_packed, np.float32(L.gate_proj.scale), osc)
                u = port.matmul_packed_m1(oq, L.up_proj.w_packed, np.float32(L.up_proj.scale), osc)
                o_inter = port.relu2_mul_into(g, u, np.empty(I, np.float32))
                got, want = _host(lib, d_inter, I, np.float32), o_inter
                if resync:
                    put(d_inter, o_inter)
            else:
                dq = linear(("down_proj",), li, (d_x,), d_inter, L.ffn_sub_norm, I, K.EPI_ADD)
                oq, osc = oracle_q(o_inter, L.ffn_sub_norm)
                ox = ox + port.matmul_packed_m1(oq, L.down_proj.w_packed, np.float32(L.down_proj.scale), osc)
                got, want = _host(lib, d_x, H, np.float32), ox
                if resync:
                    put(d_x, ox)
            diff = np.abs(dq.astype(np.int32) - oq.astype(np.int32))
            records.append((li, stage, int(np.count_nonzero(diff)), int(diff.max()),
                            float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))))
    final = _rel_l2(_host(lib, d_x, H, np.float32), ox)
    for p in (d_x, d_q, d_k, d_v, d_attn, d_inter, d_xq, d_xs, *gammas.values()):
        lib.lspk_free(p)
    return records, final


def test_every_stage_of_every_layer_on_identical_input(full, oracle, port):
    """All 120 projection stages of the first token, each fed exactly what the oracle feeds its own: the int8
    activations may differ from the oracle's only by isolated one-step rounding flips (the sum of squares is
    reduced in another order), and a stage whose activations are identical reproduces the oracle's fp32 output
    to rounding of the shared scale."""
    records, _ = _layer_walk(full, oracle, port, resync=True)
    clean = [r for r in records if r[2] == 0]
    worst = max(records, key=lambda r: r[2])
    print(f"\n[config 3, per stage on identical input] {len(clean)} of {len(records)} stages reproduce the oracle's int8 "
          f"activations exactly; the others differ in at most {worst[2]} element(s) of {2560 if worst[1] != 'down' else 6912} "
          f"(layer {worst[0]}, {worst[1]}) by {max(r[3] for r in records)} step; fp32 output of the exact stages: "
          f"max rel-L2 {max(r[4] for r in clean):.2e}; of the others: {max([r[4] for r in records if r[2]] or [0.0]):.2e}")
    assert len(records) == 120
    assert all(r[3] <= 1 for r in records), "activations may differ by one quantisation step at most"
    assert all(r[2] <= 8 for r in records), "a reordered fp32 sum moves a handful of elements, not more"
    assert len(clean) >= 90
    assert all(r[4] <= 1e-6 for r in clean)
    assert all(r[4] <= 2e-2 for r in records)


def test_first_token_layer_walk_locates_the_first_flip(full, oracle, port):
    """The same walk free-running (each stage consumes the device's own previous output): exact up to the first
    differing activation; prints where that happens and what it has grown into after 30 layers."""
    records, final = _layer_walk(full, oracle, port, resync=False)
    first = next((r for r in records if r[2]), None)
    if first is None:
        print(f"\n[config 3, first token] all {len(records)} quantised activation vectors of the 30 layers equal the "
              f"oracle's; hidden state after layer 30: rel-L2 {final:.3e}")
        assert final <= 1e-5
    else:
        li, stage, n_diff, step, _ = first
        before = records[:records.index(first)]
        print(f"\n[config 3, first token] first differing int8 activation: layer {li}, stage {stage}: {n_diff} of its "
              f"elements differ, by at most {step} step(s); hidden state after layer 30: rel-L2 {final:.3e}")
        assert step == 1, "the first difference must be a rounding flip of one step"
        assert n_diff <= 8, "a reordered fp32 sum moves a handful of elements across a rounding boundary, not more"
        assert all(r[4] <= 1e-6 for r in before), "stages before the first flip reproduce the oracle's outputs"
