"""Benchmark of the ternary-matmul hot path: tg128 decode throughput of a BitNet-2B-shaped model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the configuration the headline metric is quoted on): 30-layer BitNet-b1.58-2B-shaped
decoder with random-init ternary weights and a bf16 tied embedding, a 128-token uniform-random
prompt, then 128 greedy decode steps at batch 1 with an fp16 KV cache.  One "step" of this
benchmark is one tg128 pass: the position is rolled back to 128 and 128 tokens are decoded.
Each decoded token streams ~1.18 GB of weights (ternary projections + LM head), far more than
the 126 MB L2, so no explicit L2 flush is needed between iterations.

Prints ONE JSON line.  `value` is timed on the device (CUDA events around the 128 chained
graph launches, token fed back on the GPU).  `e2e` is the same loop driven from the host
through the public Python API: every step sends the input token from host memory and reads the
greedy token back.  `roofline` is for the dominant kernel (the ternary linear kernel), timed
live here by replaying the 120 linear launches of a token over the model's 521 MB of packed
weights.  `cpu_baseline` times the reference's own compiled CPU kernels (oracle/_ref) on the
host cores for a bounded sample of the same workload.

With --gpus N > 1 (one process per GPU under torchrun) every rank decodes its own sequence on
its own replica -- no data-path collective; torch.distributed is used only for the barrier and
the max-over-ranks of the device time.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

# The CPU legs (the reference arm, the cpu_baseline of the default arm) use every host core this process
# may run on.  torchrun exports OMP_NUM_THREADS=1 to its workers; that setting is the launcher's, not the
# user's, so it is replaced before any OpenMP runtime is loaded (numpy's included).
if os.environ.get("TORCHELASTIC_RUN_ID") or os.environ.get("OMP_NUM_THREADS") == "1":
    try:
        os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))
    except AttributeError:
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

PROMPT_LEN = 128
GEN_LEN = 128
N_STREAMS = int(os.environ.get("LSPK_BENCH_STREAMS", "8"))   # forked streams of the independent-launch GEMV measurement
METRIC = "tg128 decode tok/s at BitNet-2B shape; ternary GEMV GB/s vs B200 HBM peak"


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Sample SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        return False

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def build_model(seed: int = 0):
    entry.load_package()
    from litespark_inference_b200.torchless import synthetic
    cfg = synthetic.bitnet_2b_config()
    return cfg, synthetic.random_model(cfg, seed=seed, fast=True)


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def _set_omp_threads(n: int) -> bool:
    """Thread count of the OpenMP runtime the compiled reference kernels use (libgomp, already loaded with
    them).  Returns False when it cannot be set."""
    try:
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(int(n))
        return True
    except (OSError, AttributeError):
        return False


class CpuReference:
    """The reference's CPU path on this host: its compiled kernel objects under oracle/_ref when this CPU can
    run them (else the C restatement), driven by the oracle's numpy restatement of the reference's runtime.py
    host loop.  One prefill of the prompt (chunks of 64 rows, the reference's limit), then tg passes that roll the
    position back to the end of the prompt, exactly like the device arm."""

    def __init__(self, model, prompt, tier=None):
        self.orc = entry.load_oracle()
        tier = tier or self.orc.ref_tier()
        if tier is not None:
            self.kern, self.kind, self.what = self.orc.Kernels("ref", tier), "reference", f"oracle/_ref {tier} build"
        else:
            self.kern, self.kind = self.orc.Kernels("port"), "port"
            self.what = "oracle C restatement (no usable reference object)"
        self.model, self.prompt = model, list(prompt)
        self.threads = self.kern.max_threads()
        self.state = None

    def prefill(self, gen_len: int) -> float:
        self.state = self.orc.State(self.model.config, len(self.prompt) + gen_len + 1, np.float16)
        t0 = time.perf_counter()
        logits = self.orc.forward_prefill(self.kern, self.model, self.state, self.prompt)
        self.pp_s = time.perf_counter() - t0
        self.first = int(np.argmax(logits))
        return self.pp_s

    def tg(self, n_decode: int) -> float:
        """Seconds for n_decode greedy steps from the end of the prompt."""
        self.state.pos = len(self.prompt)
        tok = self.first
        t0 = time.perf_counter()
        for _ in range(n_decode):
            tok = int(np.argmax(self.orc.forward_one(self.kern, self.model, self.state, tok)))
        return time.perf_counter() - t0


def cpu_variants(model, prompt, n_decode: int):
    """Short samples of the other CPU configurations a user of the reference can run: its AVX2 build and a
    single OpenMP thread (tok/s over n_decode greedy steps after the full prompt)."""
    out = {}
    orc = entry.load_oracle()
    best = orc.ref_tier()
    for tier in ("avx512", "avx2"):
        if best is None or (tier == "avx512" and best != "avx512"):
            continue
        try:
            ref = CpuReference(model, prompt, tier)
            ref.prefill(n_decode)
            out[f"{tier}_all_threads_tok_s"] = n_decode / ref.tg(n_decode)
            if _set_omp_threads(1):
                n1 = max(4, n_decode // 3)
                out[f"{tier}_1_thread_tok_s"] = n1 / ref.tg(n1)
                _set_omp_threads(ref.threads)
        except (RuntimeError, OSError) as ex:
            out[f"{tier}_error"] = str(ex)[:120]
    out["sample"] = (f"{n_decode} greedy decode steps ({max(4, n_decode // 3)} on one thread) after the "
                     f"{len(prompt)}-token prompt, fp16 KV")
    return out


def run_reference_arm(args):
    """--impl reference: the reference's CPU path on the host cores, rank 0 only.  A step is one tg pass of the
    same workload as the device arm: GEN_LEN greedy steps after the PROMPT_LEN-token prompt, fp16 KV."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg, model = build_model()
    prompt = [int(t) for t in np.random.default_rng(100).integers(0, cfg.vocab_size, PROMPT_LEN)]
    ref = CpuReference(model, prompt)
    ref.prefill(GEN_LEN)
    # the whole run has to end within a few minutes: at most 12 tg passes are timed (about 3 s each); a request
    # for more steps re-uses their mean
    n_timed = min(args.steps, 12)
    n_warm = min(args.warmup, 2)
    for _ in range(n_warm):
        ref.tg(GEN_LEN)
    secs = [ref.tg(GEN_LEN) for _ in range(n_timed)]
    value = GEN_LEN * len(secs) / sum(secs)
    sample = (f"{ref.what}; every step = {GEN_LEN} greedy decode steps after the {PROMPT_LEN}-token prompt (prefilled "
              f"once, in two 64-row chunks, {ref.pp_s * 1e3:.0f} ms), fp16 KV, OMP threads={ref.threads}; "
              f"{n_timed} of the {args.steps} steps timed after {n_warm} warm-up passes")
    extra = {} if args.skip_extras else cpu_variants(model, prompt, 32)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * sum(secs) / len(secs),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic",
        "config": workload_config(1),
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": ref.threads, "kind": ref.kind, "sample": sample},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "prefill": {"tokens": PROMPT_LEN, "ms": ref.pp_s * 1e3, "tok_s": PROMPT_LEN / ref.pp_s},
        "cpu_variants": extra,
    }
    print(json.dumps(line))


def workload_config(world: int) -> dict:
    """The `config` object of the JSON line, shared by both arms so that they name the same workload."""
    return {"workload": "BitNet-2B-shaped decoder (30 layers, H=2560, I=6912, 20/5 heads, V=128256, "
                        f"bf16 tied embedding), {PROMPT_LEN}-token random prompt + {GEN_LEN} greedy steps, "
                        "batch 1 per GPU, fp16 KV",
            "parallelism": f"dp{world} (independent sequence per GPU, no collective)",
            "l2": "inputs larger than L2 (1.18 GB of weights streamed per token)",
            "step": "one tg128 pass = 128 chained decode steps",
            "arithmetic": "int8 activations x ternary (2-bit packed) weights -> int32, fp32 rescale"}


def bench_tp_mlp(dist, rank, world, model, lib, K):
    """Batch-1 MLP block (gate/up -> ReLU^2 -> SubLN+quant -> down) with the rows of gate/up/down split over
    the ranks and the fp32 slices all-gathered by NCCL, against the same block unsplit on one GPU.  A graph of
    the 30 layers' blocks is replayed; device time, max over ranks."""
    import torch
    from litespark_inference_b200.torchless import device as dev
    from litespark_inference_b200.torchless import tp
    uid = torch.zeros(128, dtype=torch.uint8, device="cuda")
    if rank == 0:
        uid = torch.tensor(list(tp.DeviceTP.make_unique_id()), dtype=torch.uint8, device="cuda")
    dist.broadcast(uid, 0)
    group = tp.DeviceTP(rank, world, bytes(uid.cpu().tolist()))
    H, I = model.config.hidden_size, model.config.intermediate_size
    W = lambda p: dev.DeviceWeight(p.w_packed, p.scale)
    sl = [[W(tp.slice_projection(getattr(L, n), world, rank)) for L in model.layers]
          for n in ("gate_proj", "up_proj", "down_proj")]
    arr = lambda ws: (ctypes.c_void_p * len(ws))(*[w.handle for w in ws])
    x = dev.DeviceArray.from_numpy(np.random.default_rng(3).standard_normal((1, H)).astype(np.float32))
    norm = dev.DeviceArray.from_numpy(np.ascontiguousarray(model.layers[0].post_attn_norm))
    sub = dev.DeviceArray.from_numpy(np.ascontiguousarray(model.layers[0].ffn_sub_norm))
    i_s, i_f = dev.DeviceArray((I // world,), np.float32), dev.DeviceArray((I,), np.float32)
    d_s, y_f = dev.DeviceArray((H // world,), np.float32), dev.DeviceArray((H,), np.float32)
    ms = ctypes.c_float(0.0)
    n_blocks, reps = len(model.layers), 20
    dist.barrier()
    K.check(lib.lspk_tp_bench_mlp(arr(sl[0]), arr(sl[1]), arr(sl[2]), n_blocks, x.ptr, norm.ptr, sub.ptr, 1e-5,
                                  i_s.ptr, i_f.ptr, d_s.ptr, y_f.ptr, reps, ctypes.byref(ms)))
    t = torch.tensor([ms.value], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    tp_us = 1000.0 * float(t.item()) / (reps * n_blocks)
    # the same graph with both gathers of every block through CUDA-IPC peer windows (plain stores + bounded waits)
    peer_us, peer_same = None, None
    try:
        handle = group.create_window(I, H)
        mine = torch.tensor(list(handle), dtype=torch.uint8, device="cuda")
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        group.open_windows([bytes(g.cpu().tolist()) for g in gathered])
        dist.barrier()
        K.check(lib.lspk_tp_bench_mlp(arr(sl[0]), arr(sl[1]), arr(sl[2]), n_blocks, x.ptr, norm.ptr, sub.ptr, 1e-5,
                                      i_s.ptr, None, d_s.ptr, None, reps, ctypes.byref(ms)))
        t = torch.tensor([ms.value], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        peer_us = 1000.0 * float(t.item()) / (reps * n_blocks)
        K.check(lib.lspk_tc_check_error())
    except Exception as ex:
        peer_us = {"error": str(ex)[:200]}
    # correctness: layer 0's block through the split path against the same block unsplit on this GPU
    group.mlp_block(sl[0][0], sl[1][0], sl[2][0], x, norm, sub, 1e-5, i_s, i_f, d_s, y_f)
    y_split = y_f.numpy()
    L0 = model.layers[0]
    full = [W(getattr(L0, n)) for n in ("gate_proj", "up_proj", "down_proj")]
    y_one = dev.DeviceArray((H,), np.float32)
    dev.linear(full[:2], [i_f, None], 1, x_f32=x, gamma=norm, epilogue=K.EPI_RELU2_MUL)
    dev.linear(full[2:], [y_one], 1, x_f32=i_f, gamma=sub)
    same = bool(np.array_equal(y_split, y_one.numpy()))
    if not isinstance(peer_us, dict):
        y_peer = group.mlp_block_peer(sl[0][0], sl[1][0], sl[2][0], x, norm, sub, 1e-5, i_s, d_s)
        peer_same = bool(np.array_equal(y_peer, y_one.numpy().reshape(-1)))
        same = same and peer_same
    flag = torch.tensor([1 if same else 0], device="cuda", dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.barrier()
    group.close()
    return {"degree": world, "us_per_mlp_block": peer_us if not isinstance(peer_us, dict) else tp_us,
            "us_per_mlp_block_nccl": tp_us, "us_per_mlp_block_peer_windows": peer_us,
            "bit_identical": bool(flag.item()),
            "how": "row-split gate/up/down slices, the two gathers of a block by plain stores into CUDA-IPC peer windows "
                   "(and, for comparison, by 2 NCCL all-gathers); graph of 30 blocks, device time, max over ranks",
            "bytes_gathered_per_block": 4 * (I + H)}


def time_linear_batch(lib, K, dev, gate_handles, up_handles, x_f32, N, reps, per_call=90):
    """Microseconds per product through lspk_linear_batch: the products (one matrix each, or gate + up pairs with
    the ReLU^2 epilogue) share one quantised activation vector and write distinct outputs; calls of up to
    `per_call` products, CUDA events around `reps` passes over all of them."""
    n = len(gate_handles)
    Kd = x_f32.shape[-1]
    xq, xs = dev.DeviceArray((1, Kd), np.int8), dev.DeviceArray((1,), np.float32)
    K.check(lib.lspk_quantize_rows(x_f32.ptr, xq.ptr, xs.ptr, 1, Kd))
    outs = dev.DeviceArray((n, N), np.float32)
    arr = (K.LinearArgs * n)()
    for i, a in enumerate(arr):
        a.w[0] = gate_handles[i]
        a.n_mats, a.epilogue = 1, K.EPI_STORE
        if up_handles is not None:
            a.w[1] = up_handles[i]
            a.n_mats, a.epilogue = 2, K.EPI_RELU2_MUL
        a.out[0] = outs.ptr + 4 * N * i
        a.M, a.prologue, a.x_i8, a.x_scales = 1, K.PRO_INT8, xq.ptr, xs.ptr
    calls = [(i, min(per_call, n - i)) for i in range(0, n, per_call)]

    def one_pass():
        for i0, cnt in calls:
            K.check(lib.lspk_linear_batch(ctypes.byref(arr[i0]), cnt))

    one_pass()
    ms = ctypes.c_float(0.0)
    K.check(lib.lspk_timer_start())
    for _ in range(reps):
        one_pass()
    K.check(lib.lspk_timer_stop(ctypes.byref(ms)))
    for d in (xq, xs, outs):
        d.free()
    return 1000.0 * float(ms.value) / (reps * n)


def measure_shape(lib, dev, K, synthetic, rng, peak, name, Ms, copies_mb=300.0):
    """One BitNet-2B projection shape at the token counts Ms: fused-quantiser linear launches rotated over
    enough device copies of the matrix to exceed the L2 (about 300 MB), as a dependency chain; for one token
    row also as independent graph nodes, in both scheduling modes of the GEMV."""
    rows = []
    N, Kd = synthetic.BITNET_2B_SHAPES[name]
    proj = synthetic.random_projection_fast(rng, N, Kd)
    n_copies = max(2, int(np.ceil(copies_mb * 1e6 / (N * Kd / 4))))
    copies = [dev.DeviceWeight(proj.w_packed, proj.scale) for _ in range(n_copies)]
    handles = (ctypes.c_void_p * n_copies)(*[c.handle for c in copies])
    for M in Ms:
        x = dev.DeviceArray.from_numpy(rng.standard_normal((M, Kd)).astype(np.float32))
        y = dev.DeviceArray((M, N), np.float32)
        ms = ctypes.c_float(0.0)
        reps = 20 if M <= 8 else 5
        K.check(lib.lspk_bench_linear_copies(handles, n_copies, x.ptr, y.ptr, M, reps, ctypes.byref(ms)))
        K.check(lib.lspk_tc_check_error())
        us = 1000.0 * ms.value / (reps * n_copies)
        nbytes = N * Kd / 4 + 4 * M * Kd + 4 * M * N
        ops = 2.0 * M * N * Kd
        row = {"shape": name, "N": N, "K": Kd, "M": M, "us": us, "GBps": nbytes / us / 1e3,
               "frac_hbm": nbytes / us / 1e3 / peak, "TOPS": ops / us / 1e6,
               "path": "tcgen05" if M >= 32 else ("mma.sync" if M > 1 else "dp4a")}
        if M == 1:
            # the same launches as independent graph nodes (forked streams): the kernel's amortised
            # throughput when it is not a link of a dependency chain.  Fused quantiser, then the reference
            # kernel's own contract (int8 vector + scale in), each in both scheduling modes.
            y8 = dev.DeviceArray((N_STREAMS, N), np.float32)
            nb8 = N * Kd / 4 + Kd + 4 * N
            for int8_in, tag, nb in ((0, "", nbytes), (1, "_int8", nb8)):
                K.check(lib.lspk_bench_linear_copies_independent(handles, None, n_copies, x.ptr, y8.ptr, 1, reps,
                                                                 N_STREAMS, int8_in, ctypes.byref(ms)))
                ui = 1000.0 * ms.value / (reps * n_copies)
                key = f"independent{tag}_launches"
                row.update({f"us_{key}": ui, f"GBps_{key}": nb / ui / 1e3, f"frac_hbm_{key}": nb / ui / 1e3 / peak})
            # the same products through the batched entry point: all copies of the matrix in one launch
            ub = time_linear_batch(lib, K, dev, [c.handle for c in copies], None, x, N, reps)
            row.update({"us_batched": ub, "GBps_batched": nb8 / ub / 1e3, "frac_hbm_batched": nb8 / ub / 1e3 / peak})
            K.check(lib.lspk_tc_check_error())
            y8.free()
        rows.append(row)
        x.free()
        y.free()
    for c in copies:
        c.free()
    return rows


def cpu_shape_medians(synthetic, rng, shapes, ms):
    """The reference's own CPU kernels at the same shapes: median microseconds of matmul_lut_{tier}_m1 (one row) and
    of the batched kernel (more rows), int8 rows in, for each compiled build, with all host threads and with one."""
    orc = entry.load_oracle()
    best = orc.ref_tier()
    tiers = [t for t in ("avx512", "avx2") if best is not None and (t != "avx512" or best == "avx512")]
    out = []
    for tier in tiers:
        kern = orc.Kernels("ref", tier)
        all_threads = kern.max_threads()
        for name in shapes:
            N, Kd = synthetic.BITNET_2B_SHAPES[name]
            proj = synthetic.random_projection_fast(rng, N, Kd)
            for M in ms:
                x = rng.standard_normal((M, Kd)).astype(np.float32)
                xq, xs = np.empty((M, Kd), np.int8), np.empty(M, np.float32)
                kern.quantize_activation_batched(x, xq, xs)
                y = np.empty((M, N), np.float32)
                row = {"build": tier, "threads": all_threads, "shape": name, "N": N, "K": Kd, "M": M}
                for threads in (all_threads, 1):
                    if not _set_omp_threads(threads):
                        continue
                    reps = 40 if M <= 8 else (8 if M <= 128 else 3)
                    times = []
                    for _ in range(reps):
                        t0 = time.perf_counter()
                        if M == 1:
                            kern.matmul_packed_m1(xq[0], proj.w_packed, proj.scale, float(xs[0]), y[0])
                        else:
                            kern.matmul_packed_mT(xq, xs, proj.w_packed, proj.scale, y)
                        times.append(time.perf_counter() - t0)
                    row["us_all_threads" if threads > 1 else "us_1_thread"] = 1e6 * statistics.median(times)
                _set_omp_threads(all_threads)
                out.append(row)
    return out


def run_sweep(args):
    """The BitNet-2B projection shapes x token counts (M = 1, 8, 32, 128, 512)."""
    entry.load_package()
    from litespark_inference_b200.torchless import device as dev
    from litespark_inference_b200.torchless import kernel as K
    from litespark_inference_b200.torchless import synthetic
    lib = K.load_library(True)
    peak, peak_kind = load_peaks()
    rng = np.random.default_rng(0)
    rows = []
    shapes = [t for t in args.sweep_shapes.split(",") if t]
    ms = tuple(int(t) for t in args.sweep_m.split(",") if t)
    for name in shapes:
        rows += measure_shape(lib, dev, K, synthetic, rng, peak, name, ms, args.sweep_mb)
    cpu = None if args.no_cpu_baseline else cpu_shape_medians(synthetic, np.random.default_rng(1), shapes, ms)
    print(json.dumps({"workload": "sweep", "peak_GBps": peak, "peak_kind": peak_kind, "rows": rows,
                      "cpu_reference_kernels": cpu}))


def run_gemv(args):
    """The single GEMV y = W x at 6912 x 2560 (the reference's own CPU-runnable kernel case): device figures as
    in the sweep, and the reference's CPU kernel on one host core (it is single-threaded at one row)."""
    entry.load_package()
    from litespark_inference_b200.torchless import device as dev
    from litespark_inference_b200.torchless import kernel as K
    from litespark_inference_b200.torchless import synthetic
    lib = K.load_library(True)
    peak, peak_kind = load_peaks()
    rng = np.random.default_rng(0)
    row = measure_shape(lib, dev, K, synthetic, rng, peak, "gate", (1,))[0]
    cpu = None
    if not args.no_cpu_baseline:
        orc = entry.load_oracle()
        tier = orc.ref_tier()
        kern, kind = (orc.Kernels("ref", tier), "reference") if tier is not None else (orc.Kernels("port"), "port")
        N, Kd = synthetic.BITNET_2B_SHAPES["gate"]
        proj = synthetic.random_projection_fast(rng, N, Kd)
        x = rng.standard_normal((1, Kd)).astype(np.float32)
        xq, xs = np.empty((1, Kd), np.int8), np.empty(1, np.float32)
        kern.quantize_activation_batched(x, xq, xs)
        times, out = [], np.empty(N, np.float32)
        for _ in range(200):
            t0 = time.perf_counter()
            kern.matmul_packed_m1(xq[0], proj.w_packed, proj.scale, float(xs[0]), out)
            times.append(time.perf_counter() - t0)
        cpu_us = 1e6 * statistics.median(times)
        cpu = {"value": cpu_us, "unit": "us per GEMV", "cores": 1, "kind": kind,
               "sample": "median of 200 calls of the one-row kernel on a 6912x2560 matrix, int8 vector in"}
    print(json.dumps({"workload": "gemv 6912x2560", "peak_GBps": peak, "peak_kind": peak_kind, "row": row,
                      "cpu_baseline": cpu}))


def run_probes(args):
    """What a decode step would gain from other ways of synchronising its ~150 stages (measurement-only kernels of
    bench_probes.cu): the kernel boundary with programmatic dependent launch, a persistent cooperative kernel with
    tagged packets or a counter barrier, and a single thread-block cluster (per-SM streaming rate, exchange cost)."""
    entry.load_package()
    from litespark_inference_b200.torchless import kernel as K
    lib = K.load_library(True)
    out = {"workload": "probes"}
    ms = ctypes.c_float(0.0)
    K.check(lib.lspk_bench_launch_floor(120, 296, 50, ctypes.byref(ms)))
    out["pdl_chain_empty_kernel_us"] = 1000.0 * ms.value / (120 * 50)
    us, cyc = ctypes.c_float(0.0), ctypes.c_double(0.0)
    for mode, name in ((0, "tagged_packets"), (1, "counter_barrier")):
        for grid in (160, 240, 296):
            K.check(lib.lspk_bench_handoff(grid, 2000, mode, ctypes.byref(us), ctypes.byref(cyc)))
            out[f"persistent_{name}_grid{grid}"] = {"us_per_round": us.value, "sm_cycles_per_round": cyc.value}
    for issuers, mode in ((1, 0), (4, 4)):          # one requesting thread per CTA, or four warps taking turns
        for cs, nc, stages in ((1, 1, 2000), (16, 1, 2000), (16, 9, 400), (1, 148, 400)):
            K.check(lib.lspk_bench_cluster(cs, nc, stages, 1, 1, mode, ctypes.byref(ms)))
            gb = cs * nc * stages * 16384 / 1e9
            out[f"stream_{nc}_clusters_of_{cs}_{issuers}_issuers"] = {"GBps_total": gb / (ms.value / 1e3),
                                                                       "GBps_per_sm": gb / (ms.value / 1e3) / (cs * nc)}
    for cs in (2, 4, 8, 16):
        K.check(lib.lspk_bench_cluster(cs, 1, 1, 2000, 1, 1, ctypes.byref(ms)))
        out[f"cluster_exchange_{cs}_ctas_us"] = 1000.0 * ms.value / 2000
    print(json.dumps(out))


def measure_hybrid(passes: int):
    """Config 5: 24-layer Mamba-2 + MoE decoder, 128 greedy steps after a 128-token prompt at batch 1 and 16
    (device time of the chained decode graph, best of `passes` + 1)."""
    entry.load_package()
    from litespark_inference_b200.torchless import hybrid as hyb
    from litespark_inference_b200.torchless import kernel as K
    lib = K.load_library(True)
    cfg = hyb.HybridConfig()
    model = hyb.random_hybrid(cfg, seed=0, fast=True)
    d = hyb.DeviceHybrid(model)
    out = {"workload": "hybrid Mamba-2 + ternary MoE decoder (24 layers, hidden 2560, 80 x 64 heads, d_state 128, 8 experts "
                       "of FFN 6912, top-2), 128-token random prompt + 128 greedy steps",
           "device_bytes": d.device_bytes, "batches": []}
    ms = ctypes.c_float(0.0)
    for B in (1, 16):
        st = hyb.HybridState(d, batch=B, max_steps=GEN_LEN)
        prompts = np.random.default_rng(7).integers(0, cfg.vocab_size, (PROMPT_LEN, B)).astype(np.int32)
        first = st.prefill(prompts)
        best = None
        for _ in range(max(passes, 1) + 1):
            K.check(lib.lspk_timer_start())
            st.decode_greedy(first, GEN_LEN)
            K.check(lib.lspk_timer_stop(ctypes.byref(ms)))
            best = ms.value if best is None else min(best, ms.value)
        out["batches"].append({"batch": B, "tok_s": B * GEN_LEN / (best / 1000.0), "ms_per_step": best / GEN_LEN,
                               "kernels_per_step": st.step_kernel_count})
        st.close()
    d.close()
    return out


def run_hybrid(args):
    print(json.dumps(measure_hybrid(args.steps)))


def main():
    global PROMPT_LEN, GEN_LEN
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-hybrid", action="store_true", help="skip the hybrid (Mamba-2 + MoE) extra measurement")
    ap.add_argument("--workload", default="tg128", choices=["tg128", "sweep", "gemv", "hybrid", "probes"],
                    help="tg128: the headline line; sweep: per-shape x token-count table of the ternary linear "
                         "kernels; gemv: the single 6912x2560 GEMV; hybrid: Mamba-2 + MoE decode (extra lines, "
                         "not the headline)")
    ap.add_argument("--sweep-shapes", default="q,k,gate,down", help="projection shapes of --workload sweep")
    ap.add_argument("--sweep-m", default="1,8,32,128,512", help="token counts of --workload sweep")
    ap.add_argument("--sweep-mb", type=float, default=300.0,
                    help="megabytes of device copies a shape is rotated over (more than the L2 by default; "
                         "smaller for profiler captures)")
    ap.add_argument("--seqs-per-gpu", type=int, default=8, help="batch of the extra data-parallel measurement")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN, help="shorter prompt for profiler captures")
    ap.add_argument("--gen-len", type=int, default=GEN_LEN, help="fewer decode steps for profiler captures")
    ap.add_argument("--skip-extras", action="store_true",
                    help="only the device-timed loop and the roofline replay (profiler captures)")
    args = ap.parse_args()
    PROMPT_LEN, GEN_LEN = args.prompt_len, args.gen_len
    if args.impl == "reference":
        run_reference_arm(args)
        return
    args.warmup = max(args.warmup, 3)
    if args.workload == "sweep":
        run_sweep(args)
        return
    if args.workload == "gemv":
        run_gemv(args)
        return
    if args.workload == "hybrid":
        run_hybrid(args)
        return
    if args.workload == "probes":
        run_probes(args)
        return

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    os.environ["LITESPARK_DEVICE"] = str(local)

    cfg, model = build_model(seed=0)
    from litespark_inference_b200.torchless import kernel as K
    from litespark_inference_b200.torchless import runtime as rt
    lib = K.load_library(True)
    dm = rt.to_device(model)
    rng = np.random.default_rng(100 + rank)
    prompt = [int(t) for t in rng.integers(0, cfg.vocab_size, PROMPT_LEN)]
    t_max = PROMPT_LEN + GEN_LEN
    state = rt.init_state(dm, t_max, kv_dtype="fp16")
    first = np.empty(1, np.int32)
    ids = np.ascontiguousarray(prompt, dtype=np.int32)
    K.check(lib.lspk_forward_prefill(state.handle, 0, ids.ctypes.data, PROMPT_LEN, None, None, first.ctypes.data))
    toks = np.empty(GEN_LEN, np.int32)
    ms = ctypes.c_float(0.0)

    def pp_device():
        state.pos = 0
        K.check(lib.lspk_timer_start())
        K.check(lib.lspk_forward_prefill(state.handle, 0, ids.ctypes.data, PROMPT_LEN, None, None, first.ctypes.data))
        K.check(lib.lspk_timer_stop(ctypes.byref(ms)))
        return float(ms.value)

    pp_device()
    pp_ms = min(pp_device() for _ in range(3))

    def tg128_device():
        state.pos = PROMPT_LEN
        K.check(lib.lspk_timer_start())
        K.check(lib.lspk_decode_greedy(state.handle, first.ctypes.data, GEN_LEN, toks.ctypes.data))
        K.check(lib.lspk_timer_stop(ctypes.byref(ms)))
        return float(ms.value)

    def barrier():
        K.check(lib.lspk_sync())
        if dist is not None:
            dist.barrier()

    for _ in range(args.warmup):
        tg128_device()
    with ClockSampler(local) as clocks:
        barrier()
        per_step = [tg128_device() for _ in range(args.steps)]
        barrier()
    total_ms = sum(per_step)
    if dist is not None:
        import torch
        t = torch.tensor([total_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    value = world * args.steps * GEN_LEN / (total_ms / 1000.0)
    step_kernels = state.step_kernel_count

    # ---- end to end through the public API: host feeds each token, reads each greedy token ----
    def tg128_host():
        state.pos = PROMPT_LEN
        tok = int(first[0])
        t0 = time.perf_counter()
        for _ in range(GEN_LEN):
            tok = rt.forward_token(state, tok)
        return time.perf_counter() - t0

    if args.skip_extras:
        args.no_cpu_baseline = True
    tg128_host()
    barrier()
    e2e_s = max(tg128_host() for _ in range(1 if args.skip_extras else max(1, min(args.steps, 3))))
    if dist is not None:
        import torch
        t = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = world * GEN_LEN / e2e_s

    # the reference API's own loop: logits [V] fp32 to the host every step, argmax on the host
    def tg128_host_logits():
        state.pos = PROMPT_LEN
        tok = int(first[0])
        t0 = time.perf_counter()
        for _ in range(GEN_LEN):
            tok = int(np.argmax(rt.forward_one(dm, state, tok)))
        return time.perf_counter() - t0

    tg128_host_logits()
    e2e_logits_value = GEN_LEN / tg128_host_logits()

    # ---- tensor-parallel variant of the MLP block (row-split gate/up/down + NCCL all-gather), N > 1 ----
    tp_info = None
    if dist is not None and not args.skip_extras:
        try:
            tp_info = bench_tp_mlp(dist, rank, world, model, lib, K)
        except Exception as ex:
            tp_info = {"error": str(ex)[:200]}

    # ---- the data-parallel serving configuration: seqs_per_gpu independent sequences per GPU in lock step, every
    #      rank its own sequences (64 sequences over 8 GPUs at the defaults), no inter-GPU traffic.  Device time,
    #      max over ranks; every sequence's tokens are then checked against the same sequence decoded alone
    #      (batch 1) on rank 0's GPU. ---------------------------------------------------------------------------
    extra = {}
    try:
        if args.skip_extras:
            raise RuntimeError("skipped (--skip-extras)")
        B = args.seqs_per_gpu
        seq_prompt = lambda g: np.ascontiguousarray(
            np.random.default_rng(500 + g).integers(0, cfg.vocab_size, PROMPT_LEN), dtype=np.int32)
        bstate = rt.init_state(dm, t_max, batch=B, kv_dtype="fp16")
        firsts = np.empty(B, np.int32)
        one = np.empty(1, np.int32)
        for b in range(B):
            pb = seq_prompt(rank * B + b)
            K.check(lib.lspk_forward_prefill(bstate.handle, b, pb.ctypes.data, PROMPT_LEN, None, None, one.ctypes.data))
            firsts[b] = one[0]
        btoks = np.empty((GEN_LEN, B), np.int32)

        def tg128_batch():
            for b in range(B):
                bstate.set_pos(b, PROMPT_LEN)
            K.check(lib.lspk_timer_start())
            K.check(lib.lspk_decode_greedy(bstate.handle, firsts.ctypes.data, GEN_LEN, btoks.ctypes.data))
            K.check(lib.lspk_timer_stop(ctypes.byref(ms)))
            return float(ms.value)

        tg128_batch()
        barrier()
        bms = min(tg128_batch() for _ in range(3))
        all_first, all_toks = [firsts.copy()], [btoks.copy()]
        if dist is not None:
            import torch
            t = torch.tensor([bms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            bms = float(t.item())
            mine = torch.tensor(np.concatenate([firsts[None, :], btoks]), device="cuda", dtype=torch.int32)
            gathered = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(gathered, mine)
            all_first = [g[0].cpu().numpy() for g in gathered]
            all_toks = [g[1:].cpu().numpy() for g in gathered]
        extra["batch8_tok_s_per_gpu"] = B * GEN_LEN / (bms / 1000.0)
        extra["config4_aggregate_tok_s"] = world * B * GEN_LEN / (bms / 1000.0)
        extra["config4"] = (f"{world * B} sequences, {B} per GPU in lock step, {PROMPT_LEN}-token prompts + {GEN_LEN} "
                            "greedy steps, device time, max over ranks")
        extra["batch8_step_kernels"] = bstate.step_kernel_count
        bstate.close()
        if rank == 0:
            same, checked = True, 0
            for r in range(world):
                for b in range(B):
                    pb = seq_prompt(r * B + b)
                    state.pos = 0
                    K.check(lib.lspk_forward_prefill(state.handle, 0, pb.ctypes.data, PROMPT_LEN, None, None, one.ctypes.data))
                    K.check(lib.lspk_decode_greedy(state.handle, one.ctypes.data, GEN_LEN, toks.ctypes.data))
                    same = same and int(one[0]) == int(all_first[r][b]) and bool(np.array_equal(toks, all_toks[r][:, b]))
                    checked += 1
            extra["dp_tokens_identical"] = same
            extra["dp_sequences_checked"] = checked
    except Exception as ex:  # the headline line must still be printed
        extra["batch8_error"] = str(ex)[:200]

    if rank != 0:
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel: the ternary linear kernel, timed live --------------------
    peak, peak_kind = load_peaks()
    n_launch, lin_bytes, lm_bytes = ctypes.c_int(0), ctypes.c_double(0.0), ctypes.c_double(0.0)
    reps = 2 if args.skip_extras else 50
    K.check(lib.lspk_bench_linears(state.handle, reps, ctypes.byref(ms), ctypes.byref(n_launch), ctypes.byref(lin_bytes)))
    lin_ms = float(ms.value) / reps
    bytes_per_launch = lin_bytes.value / n_launch.value
    us_per_launch = 1000.0 * lin_ms / n_launch.value
    lin_gbs = lin_bytes.value / (lin_ms * 1e-3) / 1e9
    K.check(lib.lspk_bench_lm_head(state.handle, 20, ctypes.byref(ms), ctypes.byref(lm_bytes)))
    lm_ms = float(ms.value) / 20
    lm_gbs = lm_bytes.value / (lm_ms * 1e-3) / 1e9
    # the single GEMV of config 0 (6912 x 2560) as independent launches: the 30 layers' gate matrices (133 MB,
    # larger than the L2) on 8 forked streams inside one graph -- what the kernel streams when it is not a link
    # of a dependency chain.  Input: the int8 vector + scale of the reference kernel's contract.  Both scheduling
    # modes, and the fused gate/up launch (two matrices, ReLU^2 epilogue) in throughput mode.
    from litespark_inference_b200.torchless import device as dev
    gate_handles = (ctypes.c_void_p * cfg.num_layers)(*[dm.projection(li, "gate_proj") for li in range(cfg.num_layers)])
    up_handles = (ctypes.c_void_p * cfg.num_layers)(*[dm.projection(li, "up_proj") for li in range(cfg.num_layers)])
    gx = dev.DeviceArray.from_numpy(np.random.default_rng(3).standard_normal((1, cfg.hidden_size)).astype(np.float32))
    gy = dev.DeviceArray((N_STREAMS, cfg.intermediate_size), np.float32)
    gemv_bytes = cfg.intermediate_size * cfg.hidden_size / 4 + cfg.hidden_size + 4 * cfg.intermediate_size
    gemv = {}
    K.check(lib.lspk_bench_linear_copies_independent(gate_handles, None, cfg.num_layers, gx.ptr, gy.ptr, 1, 20, N_STREAMS, 1,
                                                     ctypes.byref(ms)))
    us = 1000.0 * float(ms.value) / (20 * cfg.num_layers)
    gemv["launch_per_matrix"] = {"us_per_product": us, "bytes_per_product": gemv_bytes, "achieved": gemv_bytes / us / 1e3,
                                 "frac": gemv_bytes / us / 1e3 / peak,
                                 "how": f"lspk_linear per matrix, independent graph nodes on {N_STREAMS} forked streams"}
    for mname, up in (("batched", None), ("batched_gate_up", up_handles)):
        us = time_linear_batch(lib, K, dev, list(gate_handles), list(up) if up is not None else None, gx,
                               cfg.intermediate_size, 20)
        nb = gemv_bytes + (cfg.intermediate_size * cfg.hidden_size / 4 if up is not None else 0)
        gemv[mname] = {"us_per_product": us, "bytes_per_product": nb, "achieved": nb / us / 1e3, "frac": nb / us / 1e3 / peak}
    K.check(lib.lspk_tc_check_error())
    gemv_us = gemv["batched"]["us_per_product"]
    gemv_gbs = gemv["batched"]["achieved"]
    gx.free()
    gy.free()
    token_ms = total_ms / (args.steps * GEN_LEN)
    kv_bytes = 2 * cfg.num_layers * (PROMPT_LEN + GEN_LEN / 2) * cfg.num_kv_heads * 128 * 2
    token_bytes = lin_bytes.value + lm_bytes.value + kv_bytes
    token_gbs = token_bytes / (token_ms * 1e-3) / 1e9

    # ---- CPU baseline: the reference's kernels on this host's cores, bounded sample ------------------
    cpu = None
    if not args.no_cpu_baseline:
        ref = CpuReference(model, prompt)
        ref.prefill(GEN_LEN)
        n_cpu = 3
        secs = [ref.tg(GEN_LEN) for _ in range(n_cpu)]
        cpu = {"value": GEN_LEN * n_cpu / sum(secs), "unit": "tok/s", "cores": ref.threads, "kind": ref.kind,
               "sample": f"{ref.what}; {n_cpu} passes of {GEN_LEN} greedy decode steps after the {PROMPT_LEN}-token prompt "
                         f"of the same model (prefill {ref.pp_s * 1e3:.0f} ms, two 64-row chunks), fp16 KV, OMP threads={ref.threads}"}

    # ---- the hybrid configuration (extra lines, not the headline): rank 0's GPU, after the headline numbers ------
    hybrid = None
    if not args.skip_extras and not args.no_hybrid:
        try:
            state.close()
            dm.close()
            hybrid = measure_hybrid(1)
        except Exception as ex:
            hybrid = {"error": str(ex)[:200]}

    line = {
        "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic",
        "config": workload_config(world),
        "clocks": clocks.summary(),
        "e2e": {"value": e2e_value, "unit": "tok/s", "h2d_bytes_per_step": 4 * GEN_LEN,
                "d2h_bytes_per_step": 4 * GEN_LEN,
                "how": "host loop over runtime.forward_token (lspk_forward_step): token id up from pinned memory, greedy token id back, every step"},
        "e2e_logits_to_host": {"value": e2e_logits_value, "unit": "tok/s", "d2h_bytes_per_step": 4 * cfg.vocab_size * GEN_LEN,
                               "how": "forward_one returning fp32 logits [V] to the host + np.argmax, the reference API's loop"},
        "prefill": {"tokens": PROMPT_LEN, "ms": pp_ms, "tok_s": PROMPT_LEN / (pp_ms / 1000.0),
                    "how": "lspk_forward_prefill of the prompt (tcgen05 GEMM for the projections), CUDA events, best of 3"},
        "gpu_launches": args.steps * GEN_LEN * step_kernels,
        "kernels_per_token": step_kernels,
        "roofline": {"kernel": "ternary_linear_kernel (M=1, fused RMSNorm+quantiser prologue)",
                     "bound": "hbm", "achieved": lin_gbs, "peak": peak, "unit": "GB/s", "frac": lin_gbs / peak,
                     "peak_kind": f"of {peak_kind}",
                     # dram read + write per launch from the ncu capture summarised in
                     # profiles/ternary_linear_kernel_m1_bitnet2b.md (mean of the four launches of a layer)
                     "traffic": (2514944 + 1706240 + 8908800 + 4540416) / 4.0,
                     "bytes_per_launch": bytes_per_launch, "us_per_launch": us_per_launch,
                     "launches_timed": n_launch.value * reps,
                     "how": "CUDA events around graph replays of the 120 linear launches of one token over all 30 layers' weights (521 MB, > L2)"},
        "roofline_gemv_independent": {"kernel": "ternary_gemv_stream_kernel (lspk_linear_batch: one-row products, 6912x2560, int8 vector in)",
                                      "bound": "hbm", "achieved": gemv_gbs, "peak": peak, "unit": "GB/s",
                                      "frac": gemv_gbs / peak, "us_per_product": gemv_us, "bytes_per_product": gemv_bytes,
                                      "variants": gemv,
                                      "how": "the 30 layers' gate matrices (133 MB, larger than the L2) as ONE call of the batched "
                                             "entry point, CUDA events around 20 calls"},
        "roofline_lm_head": {"kernel": "lm_head_kernel<bf16>", "bound": "hbm", "achieved": lm_gbs, "peak": peak,
                             "unit": "GB/s", "frac": lm_gbs / peak, "us_per_launch": 1000.0 * lm_ms},
        "roofline_token": {"bytes_per_token": token_bytes, "us_per_token": 1000.0 * token_ms, "achieved": token_gbs,
                           "peak": peak, "unit": "GB/s", "frac": token_gbs / peak,
                           "frac_of_nominal_8TBs": token_gbs / 8000.0},
        "cpu_baseline": cpu,
        "extra": extra,
        "hybrid": hybrid,
        "tp_mlp": tp_info,
    }
    print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
