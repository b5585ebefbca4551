"""CUDA kernels against the CPU oracle and the reference-generated golden vectors, through the
C ABI (ctypes).  Integer work must be bit-exact; fp32 work either bit-exact (where the operation
sequence is identical) or within the tolerance written beside the check."""
import importlib

import numpy as np
import pytest

from tests.golden.make_golden import KERNEL_CASES, LM_CASES, ROW_CASES

pytestmark = pytest.mark.gpu

dev = importlib.import_module("litespark_inference_b200.torchless.device")
K = importlib.import_module("litespark_inference_b200.torchless.kernel")
synthetic = importlib.import_module("litespark_inference_b200.torchless.synthetic")
pack = importlib.import_module("litespark_inference_b200.torchless.pack")

SHAPES = synthetic.BITNET_2B_SHAPES
GEMV_REL_TOL = 1e-3          # stated bound on fp32 GEMV outputs


@pytest.fixture(scope="module")
def g512(golden_dir):
    return np.load(golden_dir / "kernels_avx512.npz")


def _rand_case(seed, N, Kdim, T):
    rng = np.random.default_rng(seed)
    w = rng.integers(-1, 2, (N, Kdim), dtype=np.int8)
    packed = pack.pack_ternary_4_per_byte(w)
    x = rng.standard_normal((T, Kdim)).astype(np.float32)
    ws = float(np.float32(rng.uniform(0.5, 1.5)))
    return w, packed, x, ws


# ---- (a) upload: reference layout <-> device layout ------------------------------------------
@pytest.mark.parametrize("N,Kdim", [(16, 64), (5, 20), (33, 260), (640, 2560), (2560, 6912), (17, 4), (1, 128)])
def test_upload_download_round_trip(N, Kdim):
    rng = np.random.default_rng(N * 7 + Kdim)
    packed = pack.pack_ternary_4_per_byte(rng.integers(-1, 2, (N, Kdim), dtype=np.int8))
    w = dev.DeviceWeight(packed, 1.0)
    assert np.array_equal(w.download(), packed)
    groups, chunks = (N + 15) // 16, (Kdim + 63) // 64
    assert w.device_bytes == groups * chunks * 256
    w.free()


def test_upload_rejects_bad_shapes():
    with pytest.raises(K.KernelError):
        dev.DeviceWeight(np.zeros((4, 4), np.uint8), 1.0, K=15)


# ---- drop-in entry points against the reference's golden vectors -------------------------------
@pytest.mark.parametrize("ci", range(len(KERNEL_CASES)))
def test_dropin_matmul_matches_reference_golden(g512, ci):
    packed, xq, xs = g512[f"mm{ci}_packed"], g512[f"mm{ci}_xq"], g512[f"mm{ci}_xs"]
    ws = float(g512[f"mm{ci}_wscale"])
    T = xq.shape[0]
    y = K.matmul_packed_mT(xq, xs, packed, ws)
    assert np.array_equal(y, g512[f"mm{ci}_y"])                   # same two fp32 multiplies: bit-exact
    y1 = np.stack([K.matmul_packed_m1(np.ascontiguousarray(xq[t]), packed, ws, float(xs[t])) for t in range(T)])
    assert np.array_equal(y1, g512[f"mm{ci}_y"])
    yp = K.matmul_packed_prefill(xq, packed, ws, xs)
    assert np.array_equal(yp, g512[f"mm{ci}_y"])
    acc = K.matmul_packed_mT(xq, np.ones(T, np.float32), packed, 1.0)
    assert np.array_equal(acc.astype(np.int32), g512[f"mm{ci}_acc"])


@pytest.mark.parametrize("ci", range(len(ROW_CASES)))
def test_dropin_row_helpers_match_reference_golden(g512, ci):
    g = {k.split("_", 1)[1]: g512[k] for k in g512.files if k.startswith(f"row{ci}_")}
    x = g["x"]
    T, Kd = x.shape
    xq, xs = np.empty((T, Kd), np.int8), np.empty(T, np.float32)
    K.quantize_activation_batched(x, xq, xs)
    assert np.array_equal(xq, g["xq"]) and np.array_equal(xs, g["xs"])          # bit-exact quantiser
    xq1 = np.empty(Kd, np.int8)
    s1 = K.quantize_activation(np.ascontiguousarray(x[0]), xq1)
    assert np.array_equal(xq1, g["xq"][0]) and np.float32(s1) == g["xs"][0]
    out = np.empty((T, Kd), np.float32)
    # RMSNorm: the sum of squares is reduced in another order than the 16-lane CPU loop
    assert np.allclose(K.rmsnorm_into_batched(x, g["g16"], out), g["n16"], rtol=2e-6, atol=0)
    assert np.allclose(K.rmsnorm_into_batched(x, g["g32"], out), g["n32"], rtol=2e-6, atol=0)
    o1 = np.empty(Kd, np.float32)
    assert np.allclose(K.rmsnorm_into(np.ascontiguousarray(x[0]), g["g16"], o1), g["n16"][0], rtol=2e-6, atol=0)
    rq, rs = np.empty((T, Kd), np.int8), np.empty(T, np.float32)
    K.rmsnorm_quantize_batched(x, g["g16"], rq, rs, np.empty((T, Kd), np.float32))
    assert np.allclose(rs, g["rs"], rtol=2e-6, atol=0)
    d = np.abs(rq.astype(np.int32) - g["rq"].astype(np.int32))
    assert d.max() <= 1 and (d != 0).mean() < 0.02                               # rare 1-LSB flips only
    assert np.array_equal(K.relu2_mul_into_batched(x, g["up"], out), g["r2"])    # bit-exact
    a = x[0].copy()
    assert np.array_equal(K.add_inplace(a, np.ascontiguousarray(g["up"][0])), g["add"])


@pytest.mark.parametrize("ci", range(len(LM_CASES)))
def test_dropin_lm_head_matches_reference_golden(g512, ci):
    g = {k.split("_", 1)[1]: g512[k] for k in g512.files if k.startswith(f"lm{ci}_")}
    V, H = g["e16"].shape
    x = g["x"]
    # different fp32 summation order: bound = a few ulps of the sum of |terms|
    for got, want, mag in (
        (K.lm_head_bf16(g["e16"], x, np.empty(V, np.float32)), g["l16"], 4.0),
        (K.lm_head_int8(g["e8"], g["sc"], x, np.empty(V, np.float32)), g["l8"], 127 * 0.01),
        (K.lm_head_int4(g["e4"], g["sc"], x, np.empty(V, np.float32), H), g["l4"], 8 * 0.01),
    ):
        atol = 4e-7 * mag * np.abs(x).sum()
        assert np.allclose(got, want, rtol=1e-5, atol=atol)


def test_dropin_registered_weights_and_errors():
    w, packed, x, ws = _rand_case(3, 48, 128, 1)
    xq = np.empty(128, np.int8)
    xs = K.quantize_activation(np.ascontiguousarray(x[0]), xq)
    y0 = K.matmul_packed_m1(xq, packed, ws, xs)
    K.register_packed(packed)
    y1 = K.matmul_packed_m1(xq, packed, ws, xs)
    y2 = K.matmul_packed_m1(xq, packed, 2 * ws, xs)              # scale is per call, not cached
    K.unregister_all()
    assert np.array_equal(y0, y1) and np.array_equal(y2, np.float32(2) * y0)
    # like the reference the symbol returns void; a bad shape is recorded instead of computed
    lib = K.load_library()
    lib.lspk_clear_error()
    lib.matmul_lut_m1(xq, packed, ws, xs, np.empty(48, np.float32), 48, 126)
    assert lib.lspk_error_count() == 1 and b"bad arguments" in lib.lspk_last_error()
    lib.lspk_clear_error()
    assert K.has_batched_matmul() and K.has_fused_rmsnorm_quantize() and not K.has_amx()
    assert K.max_threads() >= 100 and not K.has_omp()


# ---- device-resident linear: BitNet-2B shapes, every token count of the sweep ------------------
@pytest.mark.parametrize("name", ["q", "k", "gate", "down"])
@pytest.mark.parametrize("M", [1, 2, 3, 8, 20, 32, 128, 512])
def test_linear_int32_bit_exact_at_model_shapes(port, name, M):
    N, Kd = SHAPES[name]
    w, packed, x, ws = _rand_case(sum(map(ord, name)) * 1000 + M, N, Kd, M)
    xq, xs = np.empty((M, Kd), np.int8), np.empty(M, np.float32)
    port.quantize_activation_batched(x, xq, xs)
    want_acc = port.acc_int32(xq, packed)
    want_y = port.matmul_packed_mT(xq, xs, packed, ws)
    W = dev.DeviceWeight(packed, ws)
    # (1) pre-quantised input, the reference's kernel contract
    y, acc = dev.DeviceArray((M, N), np.float32), dev.DeviceArray((M, N), np.int32)
    dev.linear([W], [y], M, x_i8=dev.DeviceArray.from_numpy(xq), x_scales=dev.DeviceArray.from_numpy(xs),
               acc_outs=[acc])
    assert np.array_equal(acc.numpy(), want_acc)
    assert np.array_equal(y.numpy(), want_y)
    # (2) fp32 input with the quantiser fused into the kernel
    y2, acc2 = dev.DeviceArray((M, N), np.float32), dev.DeviceArray((M, N), np.int32)
    xq_t, xs_t = dev.DeviceArray((M, Kd), np.int8), dev.DeviceArray((M,), np.float32)
    dev.linear([W], [y2], M, x_f32=dev.DeviceArray.from_numpy(x), acc_outs=[acc2], xq_out=xq_t, xscale_out=xs_t)
    assert np.array_equal(xq_t.numpy(), xq) and np.array_equal(xs_t.numpy(), xs)
    assert np.array_equal(acc2.numpy(), want_acc)
    assert np.array_equal(y2.numpy(), want_y)
    rel = np.abs(y2.numpy() - want_y).max() / np.abs(want_y).max()
    assert rel <= GEMV_REL_TOL
    W.free()


@pytest.mark.parametrize("N,Kd,M", [(5, 20, 1), (33, 260, 3), (17, 64, 9), (130, 448, 5), (16, 4, 2), (1, 8, 1),
                                    (48, 12288, 1)])
def test_linear_ragged_shapes(port, N, Kd, M):
    w, packed, x, ws = _rand_case(N + Kd + M, N, Kd, M)
    xq, xs = np.empty((M, Kd), np.int8), np.empty(M, np.float32)
    port.quantize_activation_batched(x, xq, xs)
    W = dev.DeviceWeight(packed, ws)
    y, acc = dev.DeviceArray((M, N), np.float32), dev.DeviceArray((M, N), np.int32)
    xq_t = dev.DeviceArray((M, Kd), np.int8)
    dev.linear([W], [y], M, x_f32=dev.DeviceArray.from_numpy(x), acc_outs=[acc], xq_out=xq_t)
    assert np.array_equal(xq_t.numpy(), xq)            # includes the reference's scalar-tail rounding rule
    assert np.array_equal(acc.numpy(), port.acc_int32(xq, packed))
    assert np.array_equal(y.numpy(), port.matmul_packed_mT(xq, xs, packed, ws))
    W.free()


@pytest.mark.parametrize("M", [1, 4, 8, 20, 64, 160])
def test_linear_fused_qkv_norm_and_epilogues(port, M):
    """Three matrices sharing one input with the RMSNorm+quantiser prologue (q/k/v), the residual
    add epilogue (o/down) and the ReLU^2 / SiLU gates (gate/up)."""
    H, I = 2560, 6912
    rng = np.random.default_rng(40 + M)
    mats = {n: _rand_case(50 + i, *SHAPES[n], 1)[1] for i, n in enumerate(["q", "k", "v", "gate", "up"])}
    scales = {n: float(np.float32(rng.uniform(0.5, 1.5))) for n in mats}
    x = (rng.standard_normal((M, H)) * 2.0).astype(np.float32)
    gamma = synthetic.fp32_to_bf16_u16(rng.uniform(0.5, 1.5, H).astype(np.float32))
    xq, xs = np.empty((M, H), np.int8), np.empty(M, np.float32)
    port.rmsnorm_quantize_batched(x, gamma, xq, xs, np.empty((M, H), np.float32))
    dW = {n: dev.DeviceWeight(mats[n], scales[n]) for n in mats}
    dx, dg = dev.DeviceArray.from_numpy(x), dev.DeviceArray.from_numpy(gamma)
    outs = [dev.DeviceArray((M, SHAPES[n][0]), np.float32) for n in ("q", "k", "v")]
    accs = [dev.DeviceArray((M, SHAPES[n][0]), np.int32) for n in ("q", "k", "v")]
    xq_t, xs_t = dev.DeviceArray((M, H), np.int8), dev.DeviceArray((M,), np.float32)
    dev.linear([dW["q"], dW["k"], dW["v"]], outs, M, x_f32=dx, gamma=dg, acc_outs=accs, xq_out=xq_t, xscale_out=xs_t)
    got_q, got_s = xq_t.numpy(), xs_t.numpy()
    assert np.allclose(got_s, xs, rtol=2e-6, atol=0)
    d = np.abs(got_q.astype(np.int32) - xq.astype(np.int32))
    assert d.max() <= 1 and (d != 0).mean() < 0.02
    # given the activations the kernel itself produced, the integer path must be exact
    for n, a, o in zip(("q", "k", "v"), accs, outs):
        assert np.array_equal(a.numpy(), port.acc_int32(got_q, mats[n]))
        assert np.array_equal(o.numpy(), port.matmul_packed_mT(got_q, got_s, mats[n], scales[n]))
    # gated epilogues on the same input, then the residual add
    want_g = port.matmul_packed_mT(got_q, got_s, mats["gate"], scales["gate"])
    want_u = port.matmul_packed_mT(got_q, got_s, mats["up"], scales["up"])
    inter = dev.DeviceArray((M, I), np.float32)
    dev.linear([dW["gate"], dW["up"]], [inter, None], M, x_f32=dx, gamma=dg, epilogue=K.EPI_RELU2_MUL)
    want = np.empty((M, I), np.float32)
    port.relu2_mul_into_batched(want_g, want_u, want)
    assert np.array_equal(inter.numpy(), want)
    dev.linear([dW["gate"], dW["up"]], [inter, None], M, x_f32=dx, gamma=dg, epilogue=K.EPI_SILU_MUL)
    silu = (want_g / (np.exp(-want_g) + np.float32(1.0))) * want_u
    assert np.allclose(inter.numpy(), silu, rtol=1e-5, atol=1e-30)
    res = rng.standard_normal((M, SHAPES["q"][0])).astype(np.float32)
    dres = dev.DeviceArray.from_numpy(res)
    dev.linear([dW["q"]], [dres], M, x_f32=dx, gamma=dg, epilogue=K.EPI_ADD)
    assert np.array_equal(dres.numpy(), res + port.matmul_packed_mT(got_q, got_s, mats["q"], scales["q"]))


def _batch_args(items):
    """ctypes array of lspk_linear_args for lspk_linear_batch: items = [(weights, out, xq, xs, epilogue, accs)]."""
    arr = (K.LinearArgs * len(items))()
    for a, (ws_, out, xq, xs, epi, accs) in zip(arr, items):
        for i, w in enumerate(ws_):
            a.w[i] = w.handle
        for i, acc in enumerate(accs):
            a.acc_out[i] = acc.ptr
        a.out[0] = out.ptr
        a.n_mats, a.M, a.prologue, a.epilogue = len(ws_), 1, K.PRO_INT8, epi
        a.x_i8, a.x_scales = xq.ptr, xs.ptr
    return arr


def test_linear_batch_bit_exact_over_shapes(port):
    """One launch over independent one-row products of every kind the stream kernel distinguishes: the model's
    shapes, ragged K and N, a K long enough for three stages per unit, a matrix with fewer row groups than the
    grid has warps and one with many times more, each with its own activation vector; integers and floats
    against the oracle."""
    lib = K.load_library(True)
    shapes = [SHAPES["q"], SHAPES["k"], SHAPES["gate"], SHAPES["down"], (5, 20), (33, 260), (1, 8), (48, 8192),
              (7000, 1000), (16 * 1300, 64)]
    items, wants, keep = [], [], []
    for ci, (N, Kd) in enumerate(shapes):
        w, packed, x, ws = _rand_case(N * 3 + Kd, N, Kd, 1)
        xq, xs = np.empty((1, Kd), np.int8), np.empty(1, np.float32)
        port.quantize_activation_batched(x, xq, xs)
        wants.append((port.acc_int32(xq, packed), port.matmul_packed_mT(xq, xs, packed, ws)))
        W = dev.DeviceWeight(packed, ws)
        y, acc = dev.DeviceArray((1, N), np.float32), dev.DeviceArray((1, N), np.int32)
        dxq, dxs = dev.DeviceArray.from_numpy(xq), dev.DeviceArray.from_numpy(xs)
        keep.append((W, y, acc, dxq, dxs))
        items.append(([W], y, dxq, dxs, K.EPI_STORE, [acc]))
    K.check(lib.lspk_linear_batch(_batch_args(items), len(items)))
    for (W, y, acc, _, _), (want_acc, want_y), shp in zip(keep, wants, shapes):
        assert np.array_equal(acc.numpy(), want_acc), shp
        assert np.array_equal(y.numpy(), want_y), shp
    K.check(lib.lspk_tc_check_error())                     # no bounded wait of the copy rings ran out
    for W, *_ in keep:
        W.free()


def test_linear_batch_epilogues_and_argument_errors(port):
    """Gated gate/up pairs (ReLU^2 and SiLU), the residual add and plain stores mixed in one launch, against the
    one-product entry point; then what the entry point has to refuse."""
    lib = K.load_library(True)
    H, I = 2560, 6912
    rng = np.random.default_rng(321)
    mats = {n: _rand_case(250 + i, *SHAPES[n], 1)[1] for i, n in enumerate(["q", "gate", "up", "down"])}
    dW = {n: dev.DeviceWeight(mats[n], 0.5 + 0.1 * i) for i, n in enumerate(mats)}
    xh = (rng.standard_normal((1, H)) * 2.0).astype(np.float32)
    xi = rng.standard_normal((1, I)).astype(np.float32)
    qh, sh, qi, si = np.empty((1, H), np.int8), np.empty(1, np.float32), np.empty((1, I), np.int8), np.empty(1, np.float32)
    port.quantize_activation_batched(xh, qh, sh)
    port.quantize_activation_batched(xi, qi, si)
    dqh, dsh, dqi, dsi = (dev.DeviceArray.from_numpy(a) for a in (qh, sh, qi, si))
    res0 = rng.standard_normal((1, H)).astype(np.float32)

    def outputs():
        return (dev.DeviceArray((1, I), np.float32), dev.DeviceArray((1, I), np.float32),
                dev.DeviceArray.from_numpy(res0), dev.DeviceArray((1, H), np.float32))

    relu, silu, res, plain = outputs()
    items = [([dW["gate"], dW["up"]], relu, dqh, dsh, K.EPI_RELU2_MUL, []),
             ([dW["down"]], res, dqi, dsi, K.EPI_ADD, []),
             ([dW["gate"], dW["up"]], silu, dqh, dsh, K.EPI_SILU_MUL, []),
             ([dW["q"]], plain, dqh, dsh, K.EPI_STORE, [])]
    K.check(lib.lspk_linear_batch(_batch_args(items), len(items)))
    relu1, silu1, res1, plain1 = outputs()
    dev.linear([dW["gate"], dW["up"]], [relu1, None], 1, x_i8=dqh, x_scales=dsh, epilogue=K.EPI_RELU2_MUL)
    dev.linear([dW["down"]], [res1], 1, x_i8=dqi, x_scales=dsi, epilogue=K.EPI_ADD)
    dev.linear([dW["gate"], dW["up"]], [silu1, None], 1, x_i8=dqh, x_scales=dsh, epilogue=K.EPI_SILU_MUL)
    dev.linear([dW["q"]], [plain1], 1, x_i8=dqh, x_scales=dsh)
    for got, want in ((relu, relu1), (silu, silu1), (res, res1), (plain, plain1)):
        assert np.array_equal(got.numpy(), want.numpy())
    assert np.abs(res.numpy() - res0).max() > 0
    K.check(lib.lspk_tc_check_error())
    # refused: more than one row, an fp32 prologue, too many products, a gated epilogue with one matrix
    lib.lspk_clear_error()
    bad = _batch_args([([dW["q"]], plain, dqh, dsh, K.EPI_STORE, [])])
    bad[0].M = 2
    assert lib.lspk_linear_batch(bad, 1) == 1 and b"one-row" in lib.lspk_last_error()
    bad[0].M, bad[0].prologue = 1, K.PRO_QUANT
    assert lib.lspk_linear_batch(bad, 1) == 1 and b"int8 activations" in lib.lspk_last_error()
    bad[0].prologue, bad[0].epilogue = K.PRO_INT8, K.EPI_RELU2_MUL
    assert lib.lspk_linear_batch(bad, 1) == 1
    assert lib.lspk_linear_batch(bad, 0) == 1 and lib.lspk_linear_batch(bad, 1000) == 1
    lib.lspk_clear_error()


def test_bounded_wait_expiry_is_reported_and_clears(port):
    """A device-side wait that runs out sets the library's flag; the host reads it once as LSPK_ERR_DEVICE_WAIT,
    and the library keeps working (nothing faults, no kernel is left spinning)."""
    lib = K.load_library(True)
    assert lib.lspk_tc_check_error() == 0
    K.check(lib.lspk_debug_expire_wait(2000))
    assert lib.lspk_tc_check_error() == 6                   # LSPK_ERR_DEVICE_WAIT
    assert b"wait expired" in lib.lspk_last_error()
    lib.lspk_clear_error()
    assert lib.lspk_tc_check_error() == 0                   # cleared by the read
    N, Kd = 48, 256
    w, packed, x, ws = _rand_case(5, N, Kd, 1)
    xq, xs = np.empty((1, Kd), np.int8), np.empty(1, np.float32)
    port.quantize_activation_batched(x, xq, xs)
    W = dev.DeviceWeight(packed, ws)
    y = dev.DeviceArray((1, N), np.float32)
    dev.linear([W], [y], 1, x_f32=dev.DeviceArray.from_numpy(x))
    assert np.array_equal(y.numpy(), port.matmul_packed_mT(xq, xs, packed, ws))
    W.free()


def test_linear_is_linear_and_zero_safe(port):
    """Size-independent properties at the full gate/up shape: W(x1 + x2) = W x1 + W x2 on the integer
    accumulators, and an all-zero input gives exactly zero."""
    N, Kd = SHAPES["gate"]
    w, packed, _, ws = _rand_case(77, N, Kd, 1)
    rng = np.random.default_rng(78)
    a = rng.integers(-60, 61, (1, Kd), dtype=np.int8)
    b = rng.integers(-60, 61, (1, Kd), dtype=np.int8)
    W = dev.DeviceWeight(packed, ws)
    one = dev.DeviceArray.from_numpy(np.ones(1, np.float32))

    def acc_of(v):
        y, acc = dev.DeviceArray((1, N), np.float32), dev.DeviceArray((1, N), np.int32)
        dev.linear([W], [y], 1, x_i8=dev.DeviceArray.from_numpy(v), x_scales=one, acc_outs=[acc])
        return acc.numpy()

    assert np.array_equal(acc_of(a) + acc_of(b), acc_of((a + b).astype(np.int8)))
    assert not acc_of(np.zeros((1, Kd), np.int8)).any()
    assert np.array_equal(acc_of(a), (w.astype(np.int32) @ a[0].astype(np.int32))[None, :])
    y = dev.DeviceArray((1, N), np.float32)
    dev.linear([W], [y], 1, x_f32=dev.DeviceArray.from_numpy(np.zeros((1, Kd), np.float32)))
    assert not y.numpy().any()


def test_device_row_helpers_and_lm_head_rows(port):
    rng = np.random.default_rng(9)
    T, Kd, V = 5, 2560, 999
    lib = K.load_library()
    x = rng.standard_normal((T, Kd)).astype(np.float32)
    e16 = synthetic.fp32_to_bf16_u16(rng.standard_normal((V, Kd)).astype(np.float32))
    dx, de = dev.DeviceArray.from_numpy(x), dev.DeviceArray.from_numpy(e16)
    dl = dev.DeviceArray((T, V), np.float32)
    K.check(lib.lspk_lm_head(0, de.ptr, None, dx.ptr, dl.ptr, T, V, Kd))
    want = np.stack([port.lm_head_bf16(e16, np.ascontiguousarray(x[t]), np.empty(V, np.float32)) for t in range(T)])
    assert np.allclose(dl.numpy(), want, rtol=1e-5, atol=4e-7 * 4 * np.abs(x).sum(axis=1).max())
    xq, xs = dev.DeviceArray((T, Kd), np.int8), dev.DeviceArray((T,), np.float32)
    K.check(lib.lspk_quantize_rows(dx.ptr, xq.ptr, xs.ptr, T, Kd))
    wq, wsc = np.empty((T, Kd), np.int8), np.empty(T, np.float32)
    port.quantize_activation_batched(x, wq, wsc)
    assert np.array_equal(xq.numpy(), wq) and np.array_equal(xs.numpy(), wsc)


@pytest.mark.parametrize("kind,T", [(0, 2), (0, 11), (0, 16), (1, 3), (1, 9), (2, 4), (2, 16)])
def test_lm_head_many_rows_all_formats(port, kind, T):
    """Several rows of x: each warp holds a few table rows (reuse of the x values it fetched), more than
    eight rows take two passes; the vocabulary size is not a multiple of the rows a CTA covers."""
    rng = np.random.default_rng(40 + kind * 17 + T)
    Kd, V = 2560, 1001
    lib = K.load_library()
    x = rng.standard_normal((T, Kd)).astype(np.float32)
    dx = dev.DeviceArray.from_numpy(x)
    dl = dev.DeviceArray((T, V), np.float32)
    if kind == 0:
        emb = synthetic.fp32_to_bf16_u16(rng.standard_normal((V, Kd)).astype(np.float32))
        de = dev.DeviceArray.from_numpy(emb)
        K.check(lib.lspk_lm_head(0, de.ptr, None, dx.ptr, dl.ptr, T, V, Kd))
        want = np.stack([port.lm_head_bf16(emb, np.ascontiguousarray(x[t]), np.empty(V, np.float32)) for t in range(T)])
        mag = 4.0
    else:
        sc = rng.uniform(0.005, 0.02, V).astype(np.float32)
        if kind == 1:
            emb = rng.integers(-127, 128, (V, Kd), dtype=np.int8)
            want = np.stack([port.lm_head_int8(emb, sc, np.ascontiguousarray(x[t]), np.empty(V, np.float32)) for t in range(T)])
            mag = 127 * 0.02
        else:
            emb = rng.integers(0, 256, (V, Kd // 2), dtype=np.uint8)
            want = np.stack([port.lm_head_int4(emb, sc, np.ascontiguousarray(x[t]), np.empty(V, np.float32), Kd) for t in range(T)])
            mag = 8 * 0.02
        de, dsc = dev.DeviceArray.from_numpy(emb), dev.DeviceArray.from_numpy(sc)
        K.check(lib.lspk_lm_head(kind, de.ptr, dsc.ptr, dx.ptr, dl.ptr, T, V, Kd))
    assert np.allclose(dl.numpy(), want, rtol=1e-5, atol=4e-7 * mag * np.abs(x).sum(axis=1).max())


# ---- tensor-core (tcgen05) path ------------------------------------------------------------------
@pytest.mark.parametrize("N,Kd,M", [(128, 128, 32), (2560, 2560, 128), (640, 2560, 64), (6912, 2560, 512),
                                    (2560, 6912, 100), (130, 448, 33), (17, 64, 40), (300, 1000, 130)])
def test_tensor_core_path_bit_exact(port, N, Kd, M):
    """The tcgen05 int8 GEMM against the oracle and against the CUDA-core kernel: int32 accumulators
    bit-exact, fp32 outputs bit-exact (same two multiplies), at model shapes and at ragged ones
    (feature count off the 128-row tile, K off the 128-wide block, token count off the tile)."""
    lib = K.load_library()
    w, packed, x, ws = _rand_case(N * 3 + Kd + M, N, Kd, M)
    xq, xs = np.empty((M, Kd), np.int8), np.empty(M, np.float32)
    port.quantize_activation_batched(x, xq, xs)
    want_acc = port.acc_int32(xq, packed)
    want_y = port.matmul_packed_mT(xq, xs, packed, ws)
    W = dev.DeviceWeight(packed, ws)
    dxq, dxs = dev.DeviceArray.from_numpy(xq), dev.DeviceArray.from_numpy(xs)
    try:
        K.check(lib.lspk_linear_force_path(2))
        y, acc = dev.DeviceArray((M, N), np.float32), dev.DeviceArray((M, N), np.int32)
        dev.linear([W], [y], M, x_i8=dxq, x_scales=dxs, acc_outs=[acc])
        K.check(lib.lspk_tc_check_error())
        assert np.array_equal(acc.numpy(), want_acc)
        assert np.array_equal(y.numpy(), want_y)
        # fused quantiser in front, residual-add behind
        res = np.random.default_rng(1).standard_normal((M, N)).astype(np.float32)
        dres = dev.DeviceArray.from_numpy(res)
        dev.linear([W], [dres], M, x_f32=dev.DeviceArray.from_numpy(x), epilogue=K.EPI_ADD)
        K.check(lib.lspk_tc_check_error())
        assert np.array_equal(dres.numpy(), res + want_y)
        K.check(lib.lspk_linear_force_path(1))
        y1 = dev.DeviceArray((M, N), np.float32)
        dev.linear([W], [y1], M, x_i8=dxq, x_scales=dxs)
        assert np.array_equal(y1.numpy(), want_y)
    finally:
        lib.lspk_linear_force_path(0)
    W.free()
