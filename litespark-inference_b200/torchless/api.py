"""``BitNet``: the user-facing facade of the torchless runtime, GPU underneath.

Same surface as the reference's facade (litespark_inference/torchless/api.py:42-249): construction
from a model + tokenizer, ``generate`` (greedy, optionally prompt-lookup speculative, optional chat
framing, text or a ``GenResult`` with timings), ``benchmark``, ``memory_bytes``, ``kernel_paths``.
Differences that follow from the device: the model is uploaded once at construction; the plain
greedy loop runs as one graph replay per token on the device (``runtime.generate``) instead of
pulling the logits to the host each step -- the tokens are the same first-maximum argmax."""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Iterable, Optional, Union

import numpy as np

from . import kernel as _kernel
from . import runtime as _rt


@dataclass
class GenResult:
    """Returned by ``BitNet.generate(..., return_full=True)``; field names as in the reference."""
    text: str
    token_ids: list
    prompt_tokens: int
    generated_tokens: int
    prefill_seconds: float
    gen_seconds: float
    prefill_tok_per_s: float
    gen_tok_per_s: float
    speculative: bool = False
    spec_stats: Optional[dict] = None


class BitNet:
    """Torchless BitNet inference on the GPU.  Each ``generate`` call builds its own state."""

    def __init__(self, model, tokenizer, *, default_t_max: int = 2048, kv_dtype: Optional[str] = None):
        self._model = model
        self._device_model = _rt.to_device(model)
        self._tokenizer = tokenizer
        self._default_t_max = default_t_max
        self._kv_dtype = kv_dtype

    # ---- construction -----------------------------------------------------------------------------
    @classmethod
    def from_pretrained(cls, path, *, embed_dtype: str = "int4", t_max: int = 2048) -> "BitNet":
        """Load a BitNet b1.58 checkpoint from a LOCAL directory holding ``*.safetensors`` (bf16 master
        weights), ``config.json`` and ``tokenizer.json``.  Nothing is downloaded."""
        from . import loader, tokenizer as tk
        model = loader.load_bitnet_dir(path, embed_dtype=embed_dtype)
        return cls(model, tk.LocalTokenizer(path), default_t_max=t_max)

    # ---- tokenisation -----------------------------------------------------------------------------
    @property
    def tokenizer(self):
        return self._tokenizer

    @property
    def config(self):
        return self._model.config

    def encode(self, text: str) -> list:
        return self._tokenizer.encode(text)

    def decode(self, tokens: Iterable[int]) -> str:
        return self._tokenizer.decode(list(tokens))

    # ---- generation -------------------------------------------------------------------------------
    def generate(self, prompt: Union[str, list], max_new_tokens: int = 64, *, speculative: bool = False,
                 spec_k: int = 4, match_n: int = 4, return_full: bool = False,
                 chat: bool = False) -> Union[str, GenResult]:
        """Greedy decode from ``prompt`` (a string, encoded here, or a list of token ids).  Returns the
        text, or a ``GenResult`` with counts and timings when ``return_full`` is set."""
        if isinstance(prompt, str):
            text = self._tokenizer.format_chat(prompt) if chat else prompt
            prompt_ids = self._tokenizer.encode(text)
        else:
            prompt_ids = [int(t) for t in prompt]
        if not prompt_ids:
            raise ValueError("empty prompt")
        t_max = max(self._default_t_max, len(prompt_ids) + max_new_tokens + 16)
        state = _rt.init_state(self._device_model, t_max=t_max, kv_dtype=self._kv_dtype)
        spec_stats = None
        if speculative:
            # the speculative loop prefills by itself; its time is reported as generation time
            t0 = time.perf_counter()
            tokens, spec_stats = _rt.generate_speculative(self._device_model, prompt_ids, max_new_tokens,
                                                          spec_k=spec_k, match_n=match_n, state=state,
                                                          return_stats=True)
            gen_dt, prefill_dt = time.perf_counter() - t0, 0.0
        else:
            t0 = time.perf_counter()
            first = _rt.prefill_first_token(state, prompt_ids)
            prefill_dt = time.perf_counter() - t0
            t0 = time.perf_counter()
            tokens = _rt.decode_greedy(state, first, max_new_tokens) if max_new_tokens > 0 else []
            gen_dt = time.perf_counter() - t0
        state.close()
        text_out = self.decode(tokens)
        if not return_full:
            return text_out
        return GenResult(text=text_out, token_ids=list(tokens), prompt_tokens=len(prompt_ids),
                         generated_tokens=len(tokens), prefill_seconds=prefill_dt, gen_seconds=gen_dt,
                         prefill_tok_per_s=(len(prompt_ids) / prefill_dt) if prefill_dt > 0 else 0.0,
                         gen_tok_per_s=(len(tokens) / gen_dt) if gen_dt > 0 else 0.0,
                         speculative=speculative, spec_stats=spec_stats)

    # ---- benchmarking -----------------------------------------------------------------------------
    def benchmark(self, prompts: Optional[list] = None, max_new_tokens: int = 32, runs: int = 3,
                  speculative: bool = False, chat: bool = False) -> dict:
        """Repeated ``generate`` calls; the result dictionary has the reference's shape
        (``config`` / ``results`` / ``summary`` with median tok/s)."""
        if prompts is None:
            raise ValueError("pass prompts (strings or token-id lists); no built-in prompt set is shipped")
        results, all_gen, all_pre = [], [], []
        for prompt in prompts:
            gens, pres = [], []
            for _ in range(runs):
                r = self.generate(prompt, max_new_tokens, speculative=speculative, chat=chat, return_full=True)
                gens.append(r.gen_tok_per_s)
                pres.append(r.prefill_tok_per_s)
            results.append({"prompt": prompt, "gen_tok_per_s": gens, "prefill_tok_per_s": pres,
                            "median_gen": float(np.median(gens)), "median_prefill": float(np.median(pres))})
            all_gen.extend(gens)
            all_pre.extend(pres)
        return {"config": {"speculative": speculative, "max_new_tokens": max_new_tokens, "runs": runs},
                "results": results,
                "summary": {"median_gen_tok_per_s": float(np.median(all_gen)),
                            "median_prefill_tok_per_s": float(np.median(all_pre))}}

    # ---- introspection ----------------------------------------------------------------------------
    def memory_bytes(self) -> dict:
        """Stored tensor bytes per component on the host model, plus what the device copy occupies."""
        out = dict(self._model.tensor_bytes()) if hasattr(self._model, "tensor_bytes") else {}
        out["device_bytes"] = int(self._device_model.device_bytes)
        return out

    def kernel_paths(self) -> dict:
        """Which kernel library serves the calls and what it offers (the reference's keys, plus the device)."""
        try:
            return {"extension": str(_kernel.library_path()), "has_omp": _kernel.has_omp(),
                    "max_threads": _kernel.max_threads(), "has_batched_matmul": _kernel.has_batched_matmul(),
                    "has_batched_helpers": _kernel.has_batched_helpers(),
                    "has_fused_rmsnorm_quantize": _kernel.has_fused_rmsnorm_quantize(),
                    "has_amx": _kernel.has_amx(), "has_unpacked_matmul": _kernel.has_unpacked_matmul(),
                    "device": "sm_100a", "sm_count": _kernel.max_threads()}
        except Exception as e:  # same contract as the reference: report, do not raise
            return {"error": repr(e)}
