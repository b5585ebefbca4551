"""CPU oracle for the ternary-matmul hot path.  TEST INFRASTRUCTURE ONLY.

Two checkers live behind one interface:

* ``backend="port"``  -- ``oracle/_build/liboracle.so``, the plain-C restatement in
  ``oracle_kernels.c`` (always available; built by ``oracle/Makefile``).
* ``backend="ref"``   -- ``oracle/_ref/_matmul_lut_{avx512,avx2}.so``, the reference's own
  kernel sources compiled unmodified (present when the build machine had the
  reference tree; used only when the running CPU has the ISA the build needs).

On top of the kernels this module restates, in numpy, the host-side forward pass of
``litespark_inference/torchless/runtime.py`` (decode step, chunked prefill, greedy
and prompt-lookup speculative generation) so that whole-model parity can be checked
on a machine that does not have the reference tree.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this module.
The shipped library never does.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path
from typing import Optional

import numpy as np
from numpy import ctypeslib as npct

_HERE = Path(__file__).resolve().parent
_PORT_SO = _HERE / "_build" / "liboracle.so"
_REF_DIR = _HERE / "_ref"

_F32 = npct.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_I8 = npct.ndpointer(dtype=np.int8, flags="C_CONTIGUOUS")
_U8 = npct.ndpointer(dtype=np.uint8, flags="C_CONTIGUOUS")
_U16 = npct.ndpointer(dtype=np.uint16, flags="C_CONTIGUOUS")
_I32 = npct.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
_ci, _cf = ctypes.c_int, ctypes.c_float

# The reference's x86 batched kernel returns without writing when T > 64
# (matmul_lut_avx512_extern_c.cpp:256,266); drive it in chunks of at most this many rows.
REF_MAX_T = 64


def build(force: bool = False, reference_root: Optional[str] = None) -> None:
    """Run oracle/Makefile: the C restatement always; the reference's own kernel objects when a checkout of
    the reference is named (argument, or the environment variable LSPK_REFERENCE_ROOT)."""
    if force or not _PORT_SO.exists():
        subprocess.run(["make", "-C", str(_HERE), "oracle"], check=True, capture_output=True)
    ref = reference_root or os.environ.get("LSPK_REFERENCE_ROOT", "")
    if ref and Path(ref, "litespark_inference").is_dir():
        subprocess.run(["make", "-C", str(_HERE), "ref", f"REF={ref}"], check=True,
                       capture_output=True)


def _cpu_flags() -> set:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def ref_tier() -> Optional[str]:
    """Which compiled reference object this CPU can run: 'avx512', 'avx2' or None."""
    flags = _cpu_flags()
    need512 = {"avx512f", "avx512bw", "avx512dq", "avx512_vnni", "avx512vbmi", "fma"}
    if need512 <= flags and (_REF_DIR / "_matmul_lut_avx512.so").exists():
        return "avx512"
    if {"avx2", "fma"} <= flags and (_REF_DIR / "_matmul_lut_avx2.so").exists():
        return "avx2"
    return None


class Kernels:
    """Uniform access to the kernel entry points of either checker.

    Method names follow the reference's Python wrappers
    (litespark_inference/torchless/kernel.py:348-651)."""

    def __init__(self, backend: str = "port", tier: Optional[str] = None):
        if backend == "port":
            if not _PORT_SO.exists():
                build()
            self.lib = ctypes.CDLL(str(_PORT_SO))
            self.tag = None
        elif backend == "ref":
            tier = tier or ref_tier()
            if tier is None:
                raise RuntimeError("no compiled reference object usable on this CPU")
            self.lib = ctypes.CDLL(str(_REF_DIR / f"_matmul_lut_{tier}.so"))
            self.tag = tier
        else:
            raise ValueError(backend)
        self.backend = backend
        self._bind()

    def _sym(self, port_name: str, ref_name: str, argtypes, restype=None):
        fn = getattr(self.lib, port_name if self.backend == "port" else ref_name.format(T=self.tag))
        fn.argtypes = argtypes
        fn.restype = restype
        return fn

    def _bind(self):
        s = self._sym
        self._m1 = s("oracle_matmul_lut_m1", "matmul_lut_{T}_m1", [_I8, _U8, _cf, _cf, _F32, _ci, _ci])
        self._mT = s("oracle_matmul_lut_mT", "matmul_lut_{T}_mT", [_I8, _F32, _U8, _cf, _F32, _ci, _ci, _ci])
        self._quant = s("oracle_quantize_activation", "quantize_activation_{T}", [_F32, _I8, _ci], _cf)
        self._quant_b = s("oracle_quantize_activation_batched", "quantize_activation_batched_{T}",
                          [_F32, _I8, _F32, _ci, _ci])
        self._rms_bf16 = s("oracle_rmsnorm_bf16gamma", "rmsnorm_bf16gamma_fp32_{T}", [_F32, _U16, _F32, _ci, _cf])
        self._rms_f32 = s("oracle_rmsnorm_fp32gamma", "rmsnorm_fp32gamma_fp32_{T}", [_F32, _F32, _F32, _ci, _cf])
        self._rms_bf16_b = s("oracle_rmsnorm_bf16gamma_batched", "rmsnorm_bf16gamma_fp32_batched_{T}",
                             [_F32, _U16, _F32, _ci, _ci, _cf])
        self._rms_f32_b = s("oracle_rmsnorm_fp32gamma_batched", "rmsnorm_fp32gamma_fp32_batched_{T}",
                            [_F32, _F32, _F32, _ci, _ci, _cf])
        self._rmsq = s("oracle_rmsnorm_quantize_bf16gamma", "rmsnorm_quantize_bf16gamma_{T}",
                       [_F32, _U16, _I8, _F32, _ci, _cf], _cf)
        self._rmsq_b = s("oracle_rmsnorm_quantize_bf16gamma_batched", "rmsnorm_quantize_bf16gamma_batched_{T}",
                         [_F32, _U16, _I8, _F32, _F32, _ci, _ci, _cf])
        self._relu2 = s("oracle_relu2_mul", "relu2_mul_fp32_{T}", [_F32, _F32, _F32, _ci])
        self._relu2_b = s("oracle_relu2_mul_batched", "relu2_mul_fp32_batched_{T}", [_F32, _F32, _F32, _ci, _ci])
        self._add = s("oracle_add_inplace", "add_inplace_fp32_{T}", [_F32, _F32, _ci])
        self._lm_bf16 = s("oracle_lm_head_bf16", "lm_head_bf16_fp32_{T}", [_U16, _F32, _F32, _ci, _ci])
        self._lm_i8 = s("oracle_lm_head_int8", "lm_head_int8_fp32_{T}", [_I8, _F32, _F32, _F32, _ci, _ci])
        self._lm_i4 = s("oracle_lm_head_int4", "lm_head_int4_fp32_{T}", [_U8, _F32, _F32, _F32, _ci, _ci])
        self._threads = s("oracle_max_threads", "matmul_lut_{T}_max_threads", [], _ci)
        if self.backend == "port":
            self._acc = self.lib.oracle_ternary_acc_i32
            self._acc.argtypes = [_I8, _U8, _I32, _ci, _ci, _ci]
            self._acc.restype = None

    # -- matmul ------------------------------------------------------------
    def matmul_packed_m1(self, x_i8, packed_w, w_scale, x_scale, out=None):
        N, Kb = packed_w.shape
        if out is None:
            out = np.empty(N, dtype=np.float32)
        self._m1(x_i8, packed_w, w_scale, x_scale, out, N, Kb * 4)
        return out

    def matmul_packed_mT(self, x_i8, x_scales, packed_w, w_scale, out=None):
        T, K = x_i8.shape
        N, Kb = packed_w.shape
        assert Kb * 4 == K
        if out is None:
            out = np.empty((T, N), dtype=np.float32)
        if self.backend == "port":
            self._mT(x_i8, x_scales, packed_w, w_scale, out, T, N, K)
        else:
            for t0 in range(0, T, REF_MAX_T):
                t1 = min(T, t0 + REF_MAX_T)
                self._mT(np.ascontiguousarray(x_i8[t0:t1]), np.ascontiguousarray(x_scales[t0:t1]),
                         packed_w, w_scale, out[t0:t1], t1 - t0, N, K)
        return out

    def acc_int32(self, x_i8, packed_w):
        """Exact int32 accumulators W @ x for x [K] or [T, K] -> [N] or [T, N].

        With the compiled reference this is read off the fp32 output at unit scales:
        |acc| <= 127*K < 2**24 for every K used here, so float(acc) is exact."""
        x2 = np.ascontiguousarray(x_i8.reshape(-1, x_i8.shape[-1]))
        T, K = x2.shape
        N = packed_w.shape[0]
        if self.backend == "port":
            acc = np.empty((T, N), dtype=np.int32)
            self._acc(x2, packed_w, acc, T, N, K)
        else:
            assert 127 * K < 2 ** 24
            y = self.matmul_packed_mT(x2, np.ones(T, np.float32), packed_w, 1.0)
            acc = y.astype(np.int32)
            assert np.array_equal(acc.astype(np.float32), y)
        return acc.reshape(x_i8.shape[:-1] + (N,))

    # -- helpers -------------------------------------------------------------
    def quantize_activation(self, x, out_i8):
        return float(self._quant(x, out_i8, x.shape[0]))

    def quantize_activation_batched(self, x, out_i8, out_scales):
        T, K = x.shape
        self._quant_b(x, out_i8, out_scales, T, K)
        return out_scales

    def rmsnorm_into(self, x, gamma, out, eps=1e-5):
        fn = self._rms_bf16 if gamma.dtype == np.uint16 else self._rms_f32
        fn(x, gamma, out, x.shape[0], eps)
        return out

    def rmsnorm_into_batched(self, x, gamma, out, eps=1e-5):
        T, K = x.shape
        fn = self._rms_bf16_b if gamma.dtype == np.uint16 else self._rms_f32_b
        fn(x, gamma, out, T, K, eps)
        return out

    def rmsnorm_quantize_into(self, x, gamma, out_i8, tmp, eps=1e-5):
        return float(self._rmsq(x, gamma, out_i8, tmp, x.shape[0], eps))

    def rmsnorm_quantize_batched(self, x, gamma, out_i8, scales, tmp, eps=1e-5):
        T, K = x.shape
        self._rmsq_b(x, gamma, out_i8, scales, tmp, T, K, eps)
        return scales

    def relu2_mul_into(self, gate, up, out):
        self._relu2(gate, up, out, gate.shape[0])
        return out

    def relu2_mul_into_batched(self, gate, up, out):
        T, K = gate.shape
        self._relu2_b(gate, up, out, T, K)
        return out

    def add_inplace(self, a, b):
        self._add(a, b, a.shape[0])
        return a

    def lm_head_bf16(self, emb_u16, x, out):
        V, H = emb_u16.shape
        self._lm_bf16(emb_u16, x, out, V, H)
        return out

    def lm_head_int8(self, emb_i8, emb_scale, x, out):
        V, H = emb_i8.shape
        self._lm_i8(emb_i8, emb_scale, x, out, V, H)
        return out

    def lm_head_int4(self, emb_u8, emb_scale, x, out, H):
        self._lm_i4(emb_u8, emb_scale, x, out, emb_u8.shape[0], H)
        return out

    def max_threads(self) -> int:
        return int(self._threads())


# ---------------------------------------------------------------------------
# Host-side numpy restatements (load-time formats and the forward pass)
# ---------------------------------------------------------------------------

def pack_ternary(w: np.ndarray) -> np.ndarray:
    """int8 {-1,0,+1} [N,K] -> uint8 [N, ceil(K/4)]; weight k sits at bits 2*(k%4) of byte k//4,
    stored as w+1; K is zero-padded to a multiple of 4 (torchless/pack.py:16-45)."""
    assert w.dtype == np.int8 and w.ndim == 2
    N, K = w.shape
    Kp = (K + 3) // 4 * 4
    codes = np.ones((N, Kp), dtype=np.uint8)
    codes[:, :K] = (w.astype(np.int16) + 1).astype(np.uint8)
    c = codes.reshape(N, Kp // 4, 4)
    return (c[:, :, 0] | (c[:, :, 1] << 2) | (c[:, :, 2] << 4) | (c[:, :, 3] << 6)).astype(np.uint8)


def unpack_ternary(packed: np.ndarray, K: int) -> np.ndarray:
    """Inverse of pack_ternary (torchless/pack.py:48-62)."""
    N, Kb = packed.shape
    shifts = np.array([0, 2, 4, 6], dtype=np.uint8)
    codes = (packed[:, :, None] >> shifts[None, None, :]) & 3
    return (codes.reshape(N, Kb * 4).astype(np.int8) - 1)[:, :K]


def bf16_to_f32(u16: np.ndarray) -> np.ndarray:
    return (u16.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_trunc(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bits by truncation (used only to make synthetic bf16 tensors)."""
    return (np.ascontiguousarray(x, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)


def quantize_ternary_absmean(w_u16: np.ndarray, row_block: int = 128):
    """Per-tensor absmean ternary quantiser (torchless/quantize.py:24-60): scale = mean|W|
    accumulated in float64 over fp32 block sums, W_t = clip(rint(W * (1/scale)), -1, 1)."""
    N, K = w_u16.shape
    total = 0.0
    for r in range(0, N, row_block):
        total += float(np.abs(bf16_to_f32(w_u16[r:r + row_block])).sum())
    absmean = total / (N * K)
    if absmean <= 0.0:
        absmean = 1.0
    inv = 1.0 / absmean
    out = np.empty((N, K), dtype=np.int8)
    for r in range(0, N, row_block):
        out[r:r + row_block] = np.round(bf16_to_f32(w_u16[r:r + row_block]) * inv).clip(-1, 1).astype(np.int8)
    return out, absmean


def rope_tables(head_dim: int, max_pos: int, theta: float):
    """cos/sin [max_pos, D/2] in fp32 (torchless/ops.py:40-50): fp32 inv_freq, fp32 product."""
    expo = np.arange(0, head_dim, 2, dtype=np.float32) / head_dim
    inv_freq = 1.0 / (theta ** expo)
    ang = np.arange(max_pos, dtype=np.float32)[:, None] * inv_freq[None, :]
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def apply_rope(x: np.ndarray, cos_row: np.ndarray, sin_row: np.ndarray) -> np.ndarray:
    """Split-half rotation (torchless/ops.py:53-67)."""
    h = x.shape[-1] // 2
    a, b = x[..., :h], x[..., h:]
    return np.concatenate([a * cos_row - b * sin_row, a * sin_row + b * cos_row], axis=-1)


def softmax_lastdim(s: np.ndarray) -> np.ndarray:
    e = np.exp(s - s.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


class State:
    """KV cache + RoPE tables for one sequence (torchless/runtime.py:59-111).

    kv_dtype=np.float32 is the reference's cache; np.float16 models the device cache:
    values are rounded on store and widened to fp32 on use."""

    def __init__(self, cfg, t_max: int, kv_dtype=np.float32):
        D = cfg.hidden_size // cfg.num_heads
        shape = (cfg.num_layers, t_max, cfg.num_kv_heads, D)
        self.cache_k = np.zeros(shape, dtype=kv_dtype)
        self.cache_v = np.zeros(shape, dtype=kv_dtype)
        self.rope_cos, self.rope_sin = rope_tables(D, t_max, cfg.rope_theta)
        self.t_max = t_max
        self.pos = 0


def embed_row(model, token_id: int) -> np.ndarray:
    """fp32 embedding row for any storage format (torchless/runtime.py:151-168)."""
    if getattr(model, "embed_int4", None) is not None:
        b = model.embed_int4[token_id].astype(np.int8)
        row = np.empty(b.shape[0] * 2, dtype=np.float32)
        row[0::2] = ((b << 4) >> 4).astype(np.float32)
        row[1::2] = (b >> 4).astype(np.float32)
        row *= model.embed_scale[token_id]
        return row
    if getattr(model, "embed_int8", None) is not None:
        row = model.embed_int8[token_id].astype(np.float32)
        row *= model.embed_scale[token_id]
        return row
    return bf16_to_f32(model.embed_tokens[token_id:token_id + 1])[0].copy()


def _attention_rows(cfg, state: State, li: int, q_rows: np.ndarray, base_pos: int) -> np.ndarray:
    """Causal GQA attention of rows q_rows[t] (already rotated) at positions base_pos+t against
    the cache of layer li (torchless/runtime.py:230-245, 392-407).  fp32 throughout."""
    Q, KV = cfg.num_heads, cfg.num_kv_heads
    D = cfg.hidden_size // Q
    G = Q // KV
    inv = 1.0 / float(np.sqrt(D))
    out = np.empty((q_rows.shape[0], Q * D), dtype=np.float32)
    for t in range(q_rows.shape[0]):
        n = base_pos + t + 1
        kh = state.cache_k[li, :n].astype(np.float32, copy=False).transpose(1, 0, 2)   # [KV, n, D]
        vh = state.cache_v[li, :n].astype(np.float32, copy=False).transpose(1, 0, 2)
        qg = q_rows[t].reshape(KV, G, D)
        s = np.matmul(qg, kh.transpose(0, 2, 1))
        s *= inv
        p = softmax_lastdim(s)
        out[t] = np.matmul(p, vh).reshape(Q * D)
    return out


def silu_mul(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """Falcon's gate, in the reference's operation order (runtime.py:726-732): g / (exp(-g) + 1) * u."""
    out = np.negative(gate)
    np.exp(out, out=out)
    out += np.float32(1.0)
    np.divide(gate, out, out=out)
    out *= up
    return out


def lm_head(kern: Kernels, model, h: np.ndarray) -> np.ndarray:
    """LM head in whichever format the model carries: the tied embedding (runtime.py:131-148) or, for the
    Falcon-E family, its own table (runtime.py:700-706)."""
    V = model.config.vocab_size
    out = np.empty(V, dtype=np.float32)
    if getattr(model, "lm_head_int4", None) is not None:
        return kern.lm_head_int4(model.lm_head_int4, model.lm_head_scale, h, out, model.config.hidden_size)
    if getattr(model, "lm_head_int8", None) is not None:
        return kern.lm_head_int8(model.lm_head_int8, model.lm_head_scale, h, out)
    if getattr(model, "lm_head_tokens", None) is not None:
        return kern.lm_head_bf16(model.lm_head_tokens, h, out)
    if getattr(model, "embed_int4", None) is not None:
        return kern.lm_head_int4(model.embed_int4, model.embed_scale, h, out, model.config.hidden_size)
    if getattr(model, "embed_int8", None) is not None:
        return kern.lm_head_int8(model.embed_int8, model.embed_scale, h, out)
    return kern.lm_head_bf16(model.embed_tokens, h, out)


def forward_hidden(kern: Kernels, model, state: State, token_ids, trace: Optional[dict] = None) -> np.ndarray:
    """Layer loop for T >= 1 tokens starting at state.pos; returns the post-final-norm hidden
    rows [T, H] and advances state.pos.  Row by row this is the reference's decode step
    (torchless/runtime.py:171-282); for T > 1 it is its batched prefill (:285-436), which the
    reference documents to be identical per row (its fixtures agree).  Layers without sub-norms are the
    Falcon-E family (falcon_forward_one, runtime.py:735-817): the attention output and the gated product
    are quantised as they are, and the gate is SiLU."""
    c = model.config
    H, I = c.hidden_size, c.intermediate_size
    Q, KV = c.num_heads, c.num_kv_heads
    D = H // Q
    T = len(token_ids)
    if T == 0:
        raise ValueError("token_ids must be non-empty")
    if state.pos + T > state.t_max:
        raise RuntimeError(f"inference state exhausted: pos={state.pos} T={T} t_max={state.t_max}")
    eps = c.rms_norm_eps
    base = state.pos
    x = np.stack([embed_row(model, int(t)) for t in token_ids]).astype(np.float32)

    def normq(src, gamma):
        K = src.shape[1]
        q8 = np.empty((T, K), np.int8)
        sc = np.empty(T, np.float32)
        if gamma is None:
            kern.quantize_activation_batched(np.ascontiguousarray(src), q8, sc)
            return q8, sc
        tmp = np.empty((T, K), np.float32)
        if gamma.dtype == np.uint16:
            kern.rmsnorm_quantize_batched(np.ascontiguousarray(src), gamma, q8, sc, tmp, eps)
        else:
            kern.rmsnorm_into_batched(np.ascontiguousarray(src), gamma, tmp, eps)
            kern.quantize_activation_batched(tmp, q8, sc)
        return q8, sc

    def proj(q8, sc, p):
        return kern.matmul_packed_mT(q8, sc, p.w_packed, np.float32(p.scale))

    for li, L in enumerate(model.layers):
        q8, sc = normq(x, L.input_norm)
        q = proj(q8, sc, L.q_proj)
        k = proj(q8, sc, L.k_proj)
        v = proj(q8, sc, L.v_proj)
        for t in range(T):
            cr, sr = state.rope_cos[base + t], state.rope_sin[base + t]
            q[t] = apply_rope(q[t].reshape(Q, D), cr, sr).reshape(-1)
            state.cache_k[li, base + t] = apply_rope(k[t].reshape(KV, D), cr, sr)
            state.cache_v[li, base + t] = v[t].reshape(KV, D)
        attn = _attention_rows(c, state, li, q, base)
        falcon = getattr(L, "attn_sub_norm", None) is None
        q8, sc = normq(attn, None if falcon else L.attn_sub_norm)
        x += proj(q8, sc, L.o_proj)
        q8, sc = normq(x, L.post_attn_norm)
        g = proj(q8, sc, L.gate_proj)
        u = proj(q8, sc, L.up_proj)
        if falcon:
            inter = silu_mul(g, u)
        else:
            inter = np.empty((T, I), np.float32)
            kern.relu2_mul_into_batched(g, u, inter)
        q8, sc = normq(inter, None if falcon else L.ffn_sub_norm)
        x += proj(q8, sc, L.down_proj)
        if trace is not None:
            trace.setdefault("x_after_layer", []).append(x.copy())
    state.pos = base + T
    out = np.empty((T, H), np.float32)
    kern.rmsnorm_into_batched(x, model.final_norm, out, eps)
    return out


def forward_one(kern, model, state, token_id: int) -> np.ndarray:
    h = forward_hidden(kern, model, state, [int(token_id)])
    return lm_head(kern, model, np.ascontiguousarray(h[0]))


def forward_prefill(kern, model, state, token_ids, chunk: int = REF_MAX_T) -> np.ndarray:
    """Last-position logits after feeding token_ids in chunks of <= chunk rows."""
    h = None
    ids = list(token_ids)
    for i in range(0, len(ids), chunk):
        h = forward_hidden(kern, model, state, ids[i:i + chunk])
    return lm_head(kern, model, np.ascontiguousarray(h[-1]))


def forward_prefill_all_logits(kern, model, state, token_ids) -> np.ndarray:
    h = forward_hidden(kern, model, state, list(token_ids))
    return np.stack([lm_head(kern, model, np.ascontiguousarray(r)) for r in h])


def generate(kern, model, prompt, max_new_tokens: int, state: Optional[State] = None,
             kv_dtype=np.float32, return_logits: bool = False):
    """Greedy decode; np.argmax takes the first maximum (torchless/runtime.py:669-697)."""
    if state is None:
        state = State(model.config, len(prompt) + max_new_tokens, kv_dtype)
    logits = forward_prefill(kern, model, state, prompt)
    toks, all_logits = [], []
    for _ in range(max_new_tokens):
        all_logits.append(logits.copy())
        nxt = int(np.argmax(logits))
        toks.append(nxt)
        logits = forward_one(kern, model, state, nxt)
    return (toks, all_logits) if return_logits else toks


def falcon_generate(kern, model, prompt, max_new_tokens: int):
    """Greedy decode that stops before an end-of-sequence id (torchless/runtime.py:826-837); the prompt goes
    through one token at a time, as falcon_forward_prefill does (:820-824)."""
    state = State(model.config, len(prompt) + max_new_tokens + 1)
    logits = None
    for t in prompt:
        logits = forward_one(kern, model, state, int(t))
    eos = set(model.config.eos_token_ids)
    out = []
    for _ in range(max_new_tokens):
        nxt = int(np.argmax(logits))
        if nxt in eos:
            break
        out.append(nxt)
        logits = forward_one(kern, model, state, nxt)
    return out


def lookup_speculation(context, match_n: int, k: int):
    """Prompt-lookup candidates (torchless/runtime.py:492-519): longest n-gram (n from match_n
    down to 2) equal to the context's tail, latest earlier occurrence first; returns the up-to-k
    tokens that followed it."""
    L = len(context)
    if L < 2 or k <= 0:
        return []
    for n in range(min(match_n, L - 1), 1, -1):
        tail = context[L - n:]
        for i in range(L - n - 1, -1, -1):
            if context[i:i + n] == tail:
                cand = context[i + n:min(i + n + k, L)]
                if cand:
                    return cand
    return []


def generate_speculative(kern, model, prompt, max_new_tokens: int, spec_k: int = 4, match_n: int = 4,
                         eos_id: Optional[int] = None, kv_dtype=np.float32):
    """Greedy prompt-lookup speculative decode (torchless/runtime.py:522-666)."""
    state = State(model.config, len(prompt) + max_new_tokens + spec_k + 2, kv_dtype)
    logits_next = forward_prefill(kern, model, state, prompt)
    out, ctx = [], list(prompt)
    while len(out) < max_new_tokens:
        nxt = int(np.argmax(logits_next))
        if eos_id is not None and nxt == eos_id:
            break
        spec = lookup_speculation(ctx + [nxt], match_n, spec_k)
        if not spec:
            out.append(nxt)
            ctx.append(nxt)
            if len(out) >= max_new_tokens:
                break
            logits_next = forward_one(kern, model, state, nxt)
            continue
        ka = min(spec_k, len(spec), max_new_tokens - len(out))
        if ka <= 0:
            break
        start = state.pos
        lg = forward_prefill_all_logits(kern, model, state, [nxt] + spec[:ka - 1])
        accepted = 0
        bonus = None
        for i in range(ka - 1):
            pred = int(np.argmax(lg[i]))
            if pred == spec[i]:
                accepted += 1
            else:
                bonus = pred
                break
        if bonus is None:
            bonus = int(np.argmax(lg[ka - 1]))
        state.pos = start + accepted + 1
        halt = False
        for tok in [nxt] + spec[:accepted] + [bonus]:
            out.append(tok)
            ctx.append(tok)
            if (eos_id is not None and tok == eos_id) or len(out) >= max_new_tokens:
                halt = True
                break
        if halt:
            break
        logits_next = forward_one(kern, model, state, bonus)
    return out
