"""Forward pass and generation on the GPU -- the drop-in for the reference's
``litespark_inference/torchless/runtime.py``.

Same public functions, arguments and return values (``init_state``, ``forward_one``,
``forward_prefill``, ``forward_prefill_all_logits``, ``generate``, ``generate_speculative`` and the
``falcon_*`` trio), but weights, activations and the KV cache live in GPU memory and a decode step
is one CUDA-graph launch.  A host model (``model.PackedBitNetModel`` / ``PackedFalconModel``) is
uploaded on first use and the device copy is cached on the object; ``to_device`` does it
explicitly.  The host still owns tokens, positions and the speculative-decoding bookkeeping.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import numpy as np

from . import kernel as _k
from ._runtime_abi import ModelConfig
from .model import PackedBitNetModel, PackedFalconModel
from .ops import rope_tables

_PROJ = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")
_NORMS = ("input_norm", "post_attn_norm", "attn_sub_norm", "ffn_sub_norm")
_NORM_FINAL = 4


def _ptr(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


class DeviceModel:
    """GPU-resident copy of a packed model."""

    def __init__(self, host_model):
        self.lib = _k.load_library(True)
        self.config = host_model.config
        c = host_model.config
        self.is_falcon = isinstance(host_model, PackedFalconModel) or not hasattr(host_model.layers[0], "attn_sub_norm") \
            or host_model.layers[0].attn_sub_norm is None
        cfg = ModelConfig(c.hidden_size, c.num_layers, c.num_heads, c.num_kv_heads, c.intermediate_size,
                          c.vocab_size, c.rms_norm_eps, 1 if self.is_falcon else 0)
        self.handle = self.lib.lspk_model_create(ctypes.byref(cfg))
        if not self.handle:
            raise _k.KernelError(_k.last_error())
        lib, h = self.lib, self.handle
        for li, L in enumerate(host_model.layers):
            for wi, name in enumerate(_PROJ):
                p = getattr(L, name)
                if p.w_packed is None:
                    # bf16 master weights: ternarise, pack and re-tile on the device
                    w = np.ascontiguousarray(p.w_bf16, dtype=np.uint16)
                    _k.check(lib.lspk_model_set_projection_bf16(h, li, wi, _ptr(w), p.out_features, p.in_features,
                                                                float(p.scale)))
                    continue
                w = np.ascontiguousarray(p.w_packed)
                _k.check(lib.lspk_model_set_projection(h, li, wi, _ptr(w), p.out_features, p.in_features,
                                                       float(np.float32(p.scale))))
            for ni, name in enumerate(_NORMS):
                g = getattr(L, name, None)
                if g is None:
                    continue
                g = np.ascontiguousarray(g)
                _k.check(lib.lspk_model_set_norm(h, li, ni, _ptr(g), int(g.dtype == np.uint16), g.shape[0]))
        g = np.ascontiguousarray(host_model.final_norm)
        _k.check(lib.lspk_model_set_norm(h, -1, _NORM_FINAL, _ptr(g), int(g.dtype == np.uint16), g.shape[0]))
        kind, table, scale = self._table(host_model.embed_tokens, host_model.embed_int8, host_model.embed_int4,
                                         host_model.embed_scale)
        _k.check(lib.lspk_model_set_embedding(h, kind, _ptr(table), _ptr(scale)))
        if getattr(host_model, "lm_head_tokens", None) is not None or getattr(host_model, "lm_head_int8", None) is not None \
                or getattr(host_model, "lm_head_int4", None) is not None:
            kind, table, scale = self._table(host_model.lm_head_tokens, host_model.lm_head_int8,
                                             host_model.lm_head_int4, host_model.lm_head_scale)
            _k.check(lib.lspk_model_set_lm_head(h, kind, _ptr(table), _ptr(scale)))
        _k.check(lib.lspk_model_finalize(h))

    @staticmethod
    def _table(bf16, i8, i4, scale):
        if i4 is not None:
            return 2, np.ascontiguousarray(i4), np.ascontiguousarray(scale, dtype=np.float32)
        if i8 is not None:
            return 1, np.ascontiguousarray(i8), np.ascontiguousarray(scale, dtype=np.float32)
        return 0, np.ascontiguousarray(bf16), None

    @property
    def device_bytes(self) -> int:
        return int(self.lib.lspk_model_device_bytes(self.handle))

    def projection(self, layer: int, name: str):
        """Device weight handle of one projection (for lspk_linear)."""
        return self.lib.lspk_model_projection(self.handle, layer, _PROJ.index(name))

    def close(self):
        if getattr(self, "handle", None):
            self.lib.lspk_model_free(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def to_device(model) -> DeviceModel:
    """Upload (once) and return the GPU copy of a host model; a DeviceModel passes through."""
    if isinstance(model, DeviceModel):
        return model
    dm = getattr(model, "_lspk_device", None)
    if dm is None or dm.handle is None:
        dm = DeviceModel(model)
        try:
            object.__setattr__(model, "_lspk_device", dm)
        except Exception:
            pass
    return dm


def default_kv_dtype() -> str:
    """fp16 unless LITESPARK_KV_DTYPE=fp32 (the reference's cache is fp32, runtime.py:63-64)."""
    return os.environ.get("LITESPARK_KV_DTYPE", "fp16").lower()


class InferState:
    """KV cache + RoPE tables + scratch of ``batch`` sequences, on the GPU
    (reference runtime.py:59-111)."""

    def __init__(self, model, t_max: int, batch: int = 1, kv_dtype: Optional[str] = None):
        self.model = to_device(model)
        self.lib = self.model.lib
        c = self.model.config
        D = c.hidden_size // c.num_heads
        self.t_max = int(t_max)
        self.batch = int(batch)
        self.kv_dtype = (kv_dtype or default_kv_dtype()).lower()
        if self.kv_dtype not in ("fp16", "fp32"):
            raise ValueError("kv_dtype must be 'fp16' or 'fp32'")
        cos, sin = rope_tables(D, self.t_max, c.rope_theta)
        self.handle = self.lib.lspk_state_create(self.model.handle, self.t_max, self.batch,
                                                 int(self.kv_dtype == "fp16"), _ptr(cos), _ptr(sin))
        if not self.handle:
            raise _k.KernelError(_k.last_error())
        self.vocab = c.vocab_size
        # argument words of forward_token, made once (a ctypes conversion per call costs more than the call)
        self._tok_in = (ctypes.c_int * 1)()
        self._tok_out = (ctypes.c_int * 1)()

    @property
    def pos(self) -> int:
        return int(self.lib.lspk_state_get_pos(self.handle, 0))

    @pos.setter
    def pos(self, value: int) -> None:
        _k.check(self.lib.lspk_state_set_pos(self.handle, 0, int(value)))

    def get_pos(self, seq: int) -> int:
        return int(self.lib.lspk_state_get_pos(self.handle, seq))

    def set_pos(self, seq: int, value: int) -> None:
        _k.check(self.lib.lspk_state_set_pos(self.handle, seq, int(value)))

    @property
    def device_bytes(self) -> int:
        return int(self.lib.lspk_state_device_bytes(self.handle))

    @property
    def step_kernel_count(self) -> int:
        return int(self.lib.lspk_state_step_kernel_count(self.handle))

    def read_kv(self, layer: int, n_pos: int, seq: int = 0):
        c = self.model.config
        D = c.hidden_size // c.num_heads
        k = np.empty((n_pos, c.num_kv_heads, D), np.float32)
        v = np.empty((n_pos, c.num_kv_heads, D), np.float32)
        _k.check(self.lib.lspk_state_read_kv(self.handle, seq, layer, n_pos, _ptr(k), _ptr(v)))
        return k, v

    def close(self):
        if getattr(self, "handle", None):
            self.lib.lspk_state_free(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def init_state(model, t_max: int, batch: int = 1, kv_dtype: Optional[str] = None) -> InferState:
    return InferState(model, t_max, batch=batch, kv_dtype=kv_dtype)


def _raise_state(lib, rc: int):
    msg = lib.lspk_last_error().decode()
    if rc == 4:      # LSPK_ERR_STATE: the reference raises RuntimeError for an exhausted cache
        raise RuntimeError(msg)
    raise _k.KernelError(f"[{rc}] {msg}")


def forward_one(model, state: InferState, token_id: int) -> np.ndarray:
    """One decode step at ``state.pos``; returns the fp32 logits [V] (reference runtime.py:171-282)."""
    tok = np.array([int(token_id)], dtype=np.int32)
    logits = np.empty(state.vocab, dtype=np.float32)
    rc = state.lib.lspk_forward_step(state.handle, _ptr(tok), _ptr(logits), None)
    if rc:
        _raise_state(state.lib, rc)
    return logits


def forward_token(state: InferState, token_id: int) -> int:
    """One decode step of a single sequence, token id in, greedy next token id out: the step of a host loop that
    chooses its own tokens (sampling, constraints, stop strings) and needs no logits.  No copy operation and no
    stream synchronisation on this path (lspk_forward_step, one sequence, no logits)."""
    state._tok_in[0] = token_id
    rc = state.lib.lspk_forward_step(state.handle, state._tok_in, None, state._tok_out)
    if rc:
        _raise_state(state.lib, rc)
    return state._tok_out[0]


def forward_step(state: InferState, tokens, want_logits: bool = False):
    """One decode step for every sequence of a batched state: tokens [batch] -> greedy next tokens
    [batch] (and logits [batch, V] when asked)."""
    tok = np.ascontiguousarray(tokens, dtype=np.int32)
    assert tok.shape == (state.batch,)
    nxt = np.empty(state.batch, dtype=np.int32)
    logits = np.empty((state.batch, state.vocab), dtype=np.float32) if want_logits else None
    rc = state.lib.lspk_forward_step(state.handle, _ptr(tok), _ptr(logits), _ptr(nxt))
    if rc:
        _raise_state(state.lib, rc)
    return (nxt, logits) if want_logits else nxt


def forward_prefill(model, state: InferState, token_ids, seq: int = 0) -> np.ndarray:
    """Feed T prompt tokens at once; returns the last position's logits (reference runtime.py:439-456)."""
    ids = np.ascontiguousarray(list(token_ids), dtype=np.int32)
    if ids.size == 0:
        raise ValueError("token_ids must be non-empty")
    logits = np.empty(state.vocab, dtype=np.float32)
    rc = state.lib.lspk_forward_prefill(state.handle, seq, _ptr(ids), int(ids.size), _ptr(logits), None, None)
    if rc:
        _raise_state(state.lib, rc)
    return logits


def forward_prefill_all_logits(model, state: InferState, token_ids, seq: int = 0) -> np.ndarray:
    """Logits for all T positions, [T, V] (reference runtime.py:459-489)."""
    ids = np.ascontiguousarray(list(token_ids), dtype=np.int32)
    if ids.size == 0:
        raise ValueError("token_ids must be non-empty")
    out = np.empty((ids.size, state.vocab), dtype=np.float32)
    rc = state.lib.lspk_forward_prefill(state.handle, seq, _ptr(ids), int(ids.size), None, _ptr(out), None)
    if rc:
        _raise_state(state.lib, rc)
    return out


def generate(model, prompt_token_ids, max_new_tokens: int, state: Optional[InferState] = None) -> list:
    """Greedy decoding (reference runtime.py:669-697).  The prompt goes through the batched
    prefill; the decode loop then runs on the device with the argmax of each step feeding the
    next, and the generated ids come back in one copy."""
    prompt = list(prompt_token_ids)
    t_max = len(prompt) + max_new_tokens
    if state is None:
        state = init_state(model, t_max)
    elif state.t_max < t_max:
        raise ValueError(f"provided state has t_max={state.t_max}, need at least {t_max}")
    if max_new_tokens <= 0:
        forward_prefill(model, state, prompt)
        return []
    return decode_greedy(state, prefill_first_token(state, prompt), max_new_tokens)


def prefill_first_token(state: InferState, prompt_token_ids, seq: int = 0) -> int:
    """Batched prefill of the prompt; returns the greedy choice after it (first maximum), computed on
    the device -- the logits never leave it."""
    ids = np.ascontiguousarray(list(prompt_token_ids), dtype=np.int32)
    first = np.empty(1, dtype=np.int32)
    rc = state.lib.lspk_forward_prefill(state.handle, seq, _ptr(ids), int(ids.size), None, None, _ptr(first))
    if rc:
        _raise_state(state.lib, rc)
    return int(first[0])


def decode_greedy(state: InferState, first_token: int, max_new_tokens: int) -> list:
    """The greedy ids starting with ``first_token`` (already chosen after the prefill): the decode loop
    runs on the device, the argmax of each step feeding the next, and the ids come back in one copy."""
    out = [int(first_token)]
    if max_new_tokens > 1:
        # the reference's loop also runs a forward for the last generated token; only its cache
        # write is observable, and it does not change the returned ids, so stop one step earlier
        first = np.array([first_token], dtype=np.int32)
        toks = np.empty(max_new_tokens - 1, dtype=np.int32)
        rc = state.lib.lspk_decode_greedy(state.handle, _ptr(first), max_new_tokens - 1, _ptr(toks))
        if rc:
            _raise_state(state.lib, rc)
        out.extend(int(t) for t in toks)
    return out[:max(max_new_tokens, 0)]


def generate_batch(model, prompts, max_new_tokens: int, kv_dtype: Optional[str] = None) -> list:
    """Greedy decoding of several independent sequences in lock step on one GPU (one row of the
    small-batch GEMV per sequence).  All prompts are prefilled one after another; the decode loop
    is shared.  Returns one list of ids per prompt."""
    prompts = [list(p) for p in prompts]
    B = len(prompts)
    t_max = max(len(p) for p in prompts) + max_new_tokens
    state = init_state(model, t_max, batch=B, kv_dtype=kv_dtype)
    first = np.empty(B, dtype=np.int32)
    one = np.empty(1, dtype=np.int32)
    for b, p in enumerate(prompts):
        ids = np.ascontiguousarray(p, dtype=np.int32)
        rc = state.lib.lspk_forward_prefill(state.handle, b, _ptr(ids), int(ids.size), None, None, _ptr(one))
        if rc:
            _raise_state(state.lib, rc)
        first[b] = one[0]
    out = [[int(first[b])] for b in range(B)]
    if max_new_tokens > 1:
        toks = np.empty((max_new_tokens - 1, B), dtype=np.int32)
        rc = state.lib.lspk_decode_greedy(state.handle, _ptr(first), max_new_tokens - 1, _ptr(toks))
        if rc:
            _raise_state(state.lib, rc)
        for b in range(B):
            out[b].extend(int(t) for t in toks[:, b])
    state.close()
    return out


def _lookup_speculation(context: list, match_n: int, k: int) -> list:
    """Prompt-lookup candidates (reference runtime.py:492-519): the longest n-gram, n from match_n
    down to 2, that equals the context's tail and occurs earlier (latest occurrence first); returns
    up to k tokens that followed it."""
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


def generate_speculative(model, prompt_token_ids, max_new_tokens: int, spec_k: int = 4, match_n: int = 4,
                         eos_id: Optional[int] = None, state: Optional[InferState] = None,
                         return_stats: bool = False):
    """Greedy speculative decoding by prompt lookup (reference runtime.py:522-666).  Candidate
    tokens are validated in one small-batch forward; rejected positions are rolled back by resetting
    the state's position.  Output equals plain greedy decoding."""
    prompt = list(prompt_token_ids)
    t_max = len(prompt) + max_new_tokens + spec_k + 2
    if state is None:
        state = init_state(model, t_max)
    elif state.t_max < t_max:
        raise ValueError(f"state.t_max={state.t_max} < required {t_max}")
    logits_next = forward_prefill(model, state, prompt)
    generated, context = [], list(prompt)
    accept_total = step_count = matched_steps = 0
    while len(generated) < max_new_tokens:
        next_token = int(np.argmax(logits_next))
        if eos_id is not None and next_token == eos_id:
            break
        spec = _lookup_speculation(context + [next_token], match_n, spec_k)
        if not spec:
            generated.append(next_token)
            context.append(next_token)
            step_count += 1
            if len(generated) >= max_new_tokens:
                break
            logits_next = forward_one(model, state, next_token)
            continue
        k_actual = min(spec_k, len(spec), max_new_tokens - len(generated))
        if k_actual <= 0:
            break
        start_pos = state.pos
        all_logits = forward_prefill_all_logits(model, state, [next_token] + spec[:k_actual - 1])
        accepted, bonus = 0, None
        for i in range(k_actual - 1):
            pred = int(np.argmax(all_logits[i]))
            if pred == spec[i]:
                accepted += 1
            else:
                bonus = pred
                break
        if bonus is None:
            bonus = int(np.argmax(all_logits[k_actual - 1]))
        state.pos = start_pos + accepted + 1
        halt = False
        for tok in [next_token] + spec[:accepted] + [bonus]:
            generated.append(tok)
            context.append(tok)
            if (eos_id is not None and tok == eos_id) or len(generated) >= max_new_tokens:
                halt = True
                break
        if halt:
            break
        logits_next = forward_one(model, state, bonus)
        accept_total += accepted
        matched_steps += 1
        step_count += 1
    if return_stats:
        return generated, {
            "specdec_supported": True, "steps": step_count, "tokens": len(generated),
            "tokens_per_step": (len(generated) / step_count) if step_count else 0.0,
            "acceptance_rate": (accept_total / (matched_steps * (spec_k - 1))) if matched_steps and spec_k > 1 else 0.0,
            "matched_steps": matched_steps,
        }
    return generated


# ---- Falcon-E family (reference runtime.py:700-837): same device code path, arch = 1 ----------
def falcon_forward_one(model, state: InferState, token_id: int) -> np.ndarray:
    return forward_one(model, state, token_id)


def falcon_forward_prefill(model, state: InferState, token_ids) -> np.ndarray:
    return forward_prefill(model, state, token_ids)


def falcon_generate(model, token_ids, max_new_tokens: int) -> list:
    """Greedy decoding that stops at an EOS id (reference runtime.py:826-837)."""
    ids = list(token_ids)
    state = init_state(model, t_max=len(ids) + max_new_tokens + 1)
    logits = forward_prefill(model, state, ids)
    eos = set(getattr(to_device(model).config, "eos_token_ids", ()))
    out = []
    for _ in range(max_new_tokens):
        nxt = int(np.argmax(logits))
        if nxt in eos:
            break
        out.append(nxt)
        logits = forward_one(model, state, nxt)
    return out
