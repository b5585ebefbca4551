"""Forward pass at the BitNet-2B layer shape (hidden 2560, 20 query / 5 KV heads of 128, intermediate
6912) with a few layers and a small vocabulary, against the CPU oracle.

What can be asserted at this shape.  Every linear layer quantises its input to int8 after an fp32
RMSNorm; an fp32 sum that rounds one ulp differently moves an activation across a rounding boundary
with probability of a few percent per 2560-vector, and one flipped activation perturbs the following
quantisers enough to flip a few percent of theirs.  A random-init network of this width is chaotic
under that: the reference's own two x86 builds (AVX-512 and AVX2 kernels: 16-lane and 8-lane sums),
teacher-forced along the same tokens, differ by a median 0.28 in relative L2 of the logits and agree on
55 % of the greedy choices; left to themselves they emit different tokens within the first five steps
(on the toy model after 60-114 steps).  Bit-exact tokens are therefore asserted where the reference's
builds agree with each other too (the toy fixtures of test_gpu_runtime.py); here the device is held to
the band the reference's two builds keep between themselves (within a factor of 1.5: both sides are single
realisations of which activations flip), and to exactness where no activation has had a chance to flip yet.
"""
import importlib

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

rt = importlib.import_module("litespark_inference_b200.torchless.runtime")
synthetic = importlib.import_module("litespark_inference_b200.torchless.synthetic")

STEPS = 128
PROMPT = 32
MEDIAN_REL_L2_NO_REF = 0.35   # absolute fallback where the compiled reference kernels cannot run

@pytest.fixture(scope="module")
def shaped():
    cfg = synthetic.bitnet_2b_config(num_layers=3, vocab_size=4096)
    m = synthetic.random_model(cfg, seed=5, norm_jitter=0.1, fast=True)
    return cfg, m, rt.to_device(m)


def _rel_l2(got, want):
    return float(np.linalg.norm(got - want) / np.linalg.norm(want - want.mean()))


def _trajectory(oracle, kern, m, cfg, prompt, kv_dtype):
    """The oracle's greedy tokens and the logits it saw before choosing each of them."""
    toks, logits = oracle.generate(kern, m, prompt, STEPS, kv_dtype=kv_dtype, return_logits=True)
    return [int(t) for t in toks], logits


def _device_teacher_forced(dm, prompt, toks, kv):
    st = rt.init_state(dm, len(prompt) + STEPS + 1, kv_dtype=kv)
    out = [rt.forward_prefill(dm, st, prompt)]
    for t in toks[:-1]:
        out.append(rt.forward_one(dm, st, t))
    return out


def _agreement(logits, toks):
    return sum(int(np.argmax(l)) == t for l, t in zip(logits, toks)) / len(toks)


@pytest.mark.parametrize("kv", ["fp32", "fp16"])
def test_error_band_is_the_reference_builds_own(shaped, oracle, port, kv):
    """Teacher-forced over 128 decode steps, the device stays at least as close to the reference's AVX-512
    arithmetic as the reference's AVX2 build does, in logits and in greedy choices."""
    cfg, m, dm = shaped
    np_kv = np.float32 if kv == "fp32" else np.float16
    prompt = [int(t) for t in np.random.default_rng(2).integers(0, cfg.vocab_size, PROMPT)]
    try:
        k512, k2 = oracle.Kernels("ref", "avx512"), oracle.Kernels("ref", "avx2")
    except (RuntimeError, OSError):
        k512 = k2 = None
    toks, want = _trajectory(oracle, k512 or port, m, cfg, prompt, np_kv)
    got = _device_teacher_forced(dm, prompt, toks, kv)
    err = float(np.median([_rel_l2(g, w) for g, w in zip(got, want)]))
    if k2 is None:
        assert err <= MEDIAN_REL_L2_NO_REF, f"device median error {err:.3e}"
        return
    st2 = oracle.State(cfg, len(prompt) + STEPS + 1, np_kv)
    other = [oracle.forward_prefill(k2, m, st2, prompt)]
    for t in toks[:-1]:
        other.append(oracle.forward_one(k2, m, st2, t))
    band = float(np.median([_rel_l2(o, w) for o, w in zip(other, want)]))
    # Both figures are medians over one realisation of a chaotic process (which activations happen to flip), so
    # "no worse than the reference's own builds" is held to the same order of magnitude, not to the last digit.
    assert err <= 1.5 * band + 1e-3, f"device median error {err:.3e} vs the reference builds' own {band:.3e}"
    assert _agreement(got, toks) >= _agreement(other, toks) - 0.15


def test_first_positions_are_exact(shaped, oracle, port):
    """Before any activation has had a chance to flip (one or two positions), logits agree to fp32 rounding."""
    cfg, m, dm = shaped
    prompt = [int(t) for t in np.random.default_rng(3).integers(0, cfg.vocab_size, 2)]
    st, ost = rt.init_state(dm, 8, kv_dtype="fp32"), oracle.State(cfg, 8)
    for t in prompt:
        got, want = rt.forward_one(dm, st, t), oracle.forward_one(port, m, ost, t)
        assert _rel_l2(got, want) <= 1e-5


def test_long_context_at_head_dim_128(shaped, oracle, port):
    """560 positions with the fp16 cache: the decode kernel's second batch of keys at head size 128 (512 per
    batch), the prefill kernel's third.  The first decode step after the prefill must track the oracle as
    closely as the prefill itself does."""
    cfg, m, dm = shaped
    n = 560
    prompt = [int(t) for t in np.random.default_rng(9).integers(0, cfg.vocab_size, n + 2)]
    st = rt.init_state(dm, n + 4, kv_dtype="fp16")
    ost = oracle.State(cfg, n + 4, np.float16)
    e0 = _rel_l2(rt.forward_prefill(dm, st, prompt[:n]), oracle.forward_prefill(port, m, ost, prompt[:n]))
    # a single position's error is one draw from the distribution whose median the band test measures
    # (0.26-0.29 between the reference's own builds); single draws reach about twice that
    assert e0 <= 2 * MEDIAN_REL_L2_NO_REF
    for t in prompt[n:]:
        e = _rel_l2(rt.forward_one(dm, st, t), oracle.forward_one(port, m, ost, t))
        assert e <= max(2.0 * e0, 0.1) + 0.05, f"decode step error {e:.3e} vs prefill error {e0:.3e}"


@pytest.mark.parametrize("kv", ["fp16", "fp32"])
def test_batched_decode_is_bit_identical_to_single_sequences(shaped, kv):
    """A sequence's activations do not depend on what it is batched with: eight sequences of different lengths
    decoded in lock step (eight-row products, row-quantiser kernel, 128-thread attention CTAs) against each sequence
    decoded alone (one-row products with the fused quantiser, 256-thread attention CTAs), along the same tokens, at
    head size 128 and across the key counts where an attention rank goes from one key batch to two.  Compared bit
    for bit: the K and V rows every layer writes for the decoded positions (those of layer l + 1 are functions of
    layer l's attention output).  The logits come from two LM-head kernels that sum in different orders (one row:
    CUDA cores; several rows: tensor cores on a three-term bf16 split), so they are compared to 1e-5 of their
    spread and through the greedy choice."""
    cfg, m, dm = shaped
    rng = np.random.default_rng(21)
    lens = (3, 40, 17, 64, 9, 130, 33, 255)
    steps = 6
    prompts = [[int(t) for t in rng.integers(0, cfg.vocab_size, n)] for n in lens]
    forced = rng.integers(0, cfg.vocab_size, (steps, len(lens))).astype(np.int32)
    t_max = max(lens) + steps + 1
    B = len(lens)
    st = rt.init_state(dm, t_max, batch=B, kv_dtype=kv)
    for b, p in enumerate(prompts):
        ids = np.ascontiguousarray(p, dtype=np.int32)
        assert st.lib.lspk_forward_prefill(st.handle, b, ids.ctypes.data, int(ids.size), None, None, None) == 0
    together = [rt.forward_step(st, forced[i], want_logits=True)[1].copy() for i in range(steps)]
    kv_together = [[st.read_kv(li, lens[b] + steps, seq=b) for li in range(cfg.num_layers)] for b in range(B)]
    st.close()
    for b, p in enumerate(prompts):
        s1 = rt.init_state(dm, t_max, kv_dtype=kv)
        rt.forward_prefill(dm, s1, p)
        for i in range(steps):
            alone = rt.forward_one(dm, s1, int(forced[i, b]))
            spread = float(alone.max() - alone.min())
            assert np.abs(alone - together[i][b]).max() <= 1e-5 * spread, (b, i)
            assert int(np.argmax(alone)) == int(np.argmax(together[i][b])), (b, i)
        for li in range(cfg.num_layers):
            k1, v1 = s1.read_kv(li, lens[b] + steps)
            k8, v8 = kv_together[b][li]
            assert np.array_equal(k1.view(np.uint32), k8.view(np.uint32)), (b, li)
            assert np.array_equal(v1.view(np.uint32), v8.view(np.uint32)), (b, li)
        s1.close()
