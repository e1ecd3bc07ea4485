"""A thin, optional wrapper over a model folder's tokenizer.json.

The reference's Python package exposes a `Tokenizer` (tests/test_rvllm_python.py:1-5) and its
evaluation binary reads tokenizer.json (v3/crates/rvllm-bench/src/bin/rvllm_eval.rs:57-83).
The engine itself works on token ids; text is a convenience that needs the `tokenizers`
package and a tokenizer.json.
"""
from __future__ import annotations

import os
from typing import List, Optional

from .errors import ConfigError


class Tokenizer:
    def __init__(self, path: str):
        try:
            from tokenizers import Tokenizer as _Tok
        except ImportError:
            raise ConfigError("the `tokenizers` package is not installed; pass token ids instead of text") from None
        self._tok = _Tok.from_file(path)

    @classmethod
    def from_model_dir(cls, model_dir: str, required: bool = True) -> Optional["Tokenizer"]:
        path = os.path.join(model_dir, "tokenizer.json")
        if not os.path.exists(path):
            if required:
                raise ConfigError(f"no tokenizer.json in {model_dir}")
            return None
        try:
            return cls(path)
        except ConfigError:
            if required:
                raise
            return None

    def encode(self, text: str) -> List[int]:
        return list(self._tok.encode(text).ids)

    def decode(self, ids) -> str:
        return self._tok.decode(list(ids))
