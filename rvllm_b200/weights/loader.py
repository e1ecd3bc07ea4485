"""Binding checkpoint tensors to a model by tensor name.

The model says which tensors it expects (name -> shape); the folder says which it has.
Everything that does not match is reported in ONE `LoaderError`: missing tensors,
unexpected tensors and wrong shapes together (the reference raises per tensor,
v3/crates/rvllm-loader/src/load.rs:321-332, and has the ShapeMismatch variant,
rvllm-core/src/error.rs:196-200, without ever raising it).

Dtype rule: with a bfloat16 engine, 16-bit float tensors are kept as bfloat16 and tensors
stored in 32 bits stay 32-bit; integer tables become int32; with a float32 engine every
float tensor becomes float32.
"""
from __future__ import annotations

import fnmatch
from typing import Dict, Iterable, Tuple

import torch

from ..errors import LoaderError
from .safetensors_io import open_model_files, TensorEntry


def engine_dtype_of(stored: torch.dtype, engine_dtype: torch.dtype) -> torch.dtype:
    if stored in (torch.int32, torch.int64):
        return torch.int32
    if engine_dtype == torch.float32:
        return torch.float32
    if stored == torch.float32:
        return torch.float32
    return torch.bfloat16


_NAME_TO_TORCH = {"F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
                  "I32": torch.int32, "I64": torch.int64}


class WeightSource:
    """The tensors of a model folder, checked against what a model expects."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self.entries: Dict[str, TensorEntry] = open_model_files(model_dir)

    def check(self, expected: Dict[str, Tuple[int, ...]], ignored: Iterable[str] = ()) -> None:
        ignored = tuple(ignored)
        missing = [n for n in expected if n not in self.entries]
        unexpected = [n for n in self.entries if n not in expected
                      and not any(fnmatch.fnmatch(n, pat) for pat in ignored)]
        wrong = [f"{n}: expected {list(expected[n])}, file has {list(self.entries[n].shape)}"
                 for n in expected if n in self.entries and tuple(self.entries[n].shape) != tuple(expected[n])]
        if missing or unexpected or wrong:
            raise LoaderError("checkpoint tensors do not match the model", path=self.model_dir,
                              missing=sorted(missing), unexpected=sorted(unexpected), wrong_shape=sorted(wrong))

    def get(self, name: str, engine_dtype: torch.dtype, device) -> torch.Tensor:
        e = self.entries[name]
        t = e.file.tensor(name)
        target = engine_dtype_of(_NAME_TO_TORCH[e.dtype], engine_dtype)
        return t.to(device=device, dtype=target, copy=True).contiguous()
