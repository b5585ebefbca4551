"""Tokenizer access for the BitNet facade.

Mirrors what the reference's facade needs from its tokenizer object (``encode``, ``decode``,
``format_chat``; litespark_inference/torchless/api.py:81-88, 109-113).  Text handling is host-side and
unrelated to the GPU path: this module only wraps a local ``tokenizer.json`` with the ``tokenizers``
package when both are present; nothing is downloaded."""
from __future__ import annotations

from pathlib import Path
from typing import Iterable, List


class LocalTokenizer:
    """``tokenizer.json`` on disk, through the ``tokenizers`` package."""

    def __init__(self, path):
        try:
            from tokenizers import Tokenizer
        except ImportError as exc:  # pragma: no cover - depends on the environment
            raise RuntimeError("the 'tokenizers' package is needed to read tokenizer.json") from exc
        p = Path(path)
        if p.is_dir():
            p = p / "tokenizer.json"
        if not p.exists():
            raise FileNotFoundError(f"no tokenizer.json at {p} (this build never downloads one)")
        self._tok = Tokenizer.from_file(str(p))

    def encode(self, text: str) -> List[int]:
        return list(self._tok.encode(text).ids)

    def decode(self, tokens: Iterable[int]) -> str:
        return self._tok.decode(list(tokens))

    @staticmethod
    def format_chat(user_text: str) -> str:
        """Single-turn chat framing of the BitNet instruct checkpoints."""
        return f"User: {user_text}<|eot_id|>Assistant: "


class IdTokenizer:
    """Stand-in for runs without any tokenizer file: text is a space-separated list of token ids."""

    def encode(self, text: str) -> List[int]:
        return [int(t) for t in text.split()]

    def decode(self, tokens: Iterable[int]) -> str:
        return " ".join(str(int(t)) for t in tokens)

    @staticmethod
    def format_chat(user_text: str) -> str:
        return user_text
