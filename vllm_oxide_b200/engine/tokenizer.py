"""Text <-> token ids, from a model folder's tokenizer.json (optional: the engine speaks ids).

The reference reads `<model_dir>/tokenizer.json` with the `tokenizers` library; encoding adds
the special tokens that the file's post-processor defines (a leading BOS for Llama 3), decoding
skips special tokens (crates/engine/src/tokenizer.rs:14-39). Same library, same two calls here.
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence

from ..errors import EngineError


class TokenizerError(EngineError):
    """tokenizer.json cannot be read, or a text cannot be encoded / ids decoded."""


class TextTokenizer:
    def __init__(self, inner):
        self._inner = inner

    @classmethod
    def load(cls, model_dir: str) -> Optional["TextTokenizer"]:
        """The tokenizer of a model folder; None if the folder has no tokenizer.json."""
        path = os.path.join(model_dir, "tokenizer.json")
        if not os.path.exists(path):
            return None
        try:
            from tokenizers import Tokenizer
        except ImportError as e:
            raise TokenizerError(f"{path}: the 'tokenizers' package is needed to read it: {e}") from e
        try:
            return cls(Tokenizer.from_file(path))
        except Exception as e:                      # the library raises a bare Exception on a malformed file
            raise TokenizerError(f"{path}: {e}") from e

    def encode(self, text: str) -> List[int]:
        """Token ids of `text`, special tokens of the post-processor added (BOS first)."""
        try:
            return list(self._inner.encode(text, add_special_tokens=True).ids)
        except Exception as e:
            raise TokenizerError(str(e)) from e

    def decode(self, ids: Sequence[int]) -> str:
        """Text of `ids`, special tokens (BOS, EOS) skipped."""
        try:
            return self._inner.decode([int(i) for i in ids], skip_special_tokens=True)
        except Exception as e:
            raise TokenizerError(str(e)) from e
