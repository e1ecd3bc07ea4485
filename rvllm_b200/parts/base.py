"""Interfaces of the parts a layer is put together from, and their registries.

A part is built from parameters only (sizes and constants; never a model's name), says which
tensors it owns (`tensor_specs`, names relative to its prefix) and receives them through
`bind`.  Kinds of part and what each must offer:

* position encoding: `prepare(max_len, device)`; `rotation_tables()` -> (cos, sin) float
  tables [max_len, rotary_dim/2] or None; `on_embeddings(x, ctx)` -> x for encodings that act
  on the input of the first layer.
* norm: `__call__(x, ctx)` -> tensor of the same shape.
* mixer: `cache_need()` -> `KvCacheNeed`, `StateNeed` or None;
  `__call__(x, ctx, cache, residual, write_cache)` -> residual + mixed x.  `cache` is the
  `CacheView` of the run entry's cache slot.
* feed-forward: `__call__(x, ctx, residual)` -> residual + f(x).
* block: built from `parts`, the layer's built parts by role name (which roles it needs is the
  block's own matter), plus its parameters; `__call__(x, ctx, cache, write_cache)` -> x.
* hook: `__call__(x, ctx)` -> x, on the embedded tokens or on the float32 logits.

A part whose step cannot be recorded into a CUDA graph (it reads device values on the host, or
launches a number of kernels that depends on the data) sets `graph_safe = False`; a model with
such a part runs its decode steps eagerly.

`ctx` is the step's `StepContext` (tokens' positions, the attention metadata of each cache
group, state slots, the kernel library).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional, Tuple

import torch


@dataclass(frozen=True)
class TensorSpec:
    shape: Tuple[int, ...]
    init: str          # "matrix", "norm" or "bias": which random distribution fills it


@dataclass(frozen=True)
class KvCacheNeed:
    """Paged keys and values; `window` None keeps every key, W keeps the last W."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """State of fixed size per request (shape without the request dimension)."""
    shape: Tuple[int, ...]
    dtype: str = "float32"


class Part:
    graph_safe = True      # whether the part's work in a decode step may be captured in a CUDA graph

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {}

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        """`get(name)` returns the device tensor stored under the part's prefix + name."""


class Registry:
    def __init__(self, what: str):
        self.what = what
        self._items: Dict[str, Callable[..., Any]] = {}

    def register(self, kind: str, factory: Callable[..., Any]) -> None:
        self._items[kind] = factory

    def unregister(self, kind: str) -> None:
        self._items.pop(kind, None)

    def build(self, kind: str, **params):
        if kind not in self._items:
            from ..errors import ConfigError
            raise ConfigError(f"unknown {self.what} {kind!r}; known: {', '.join(sorted(self._items))}")
        return self._items[kind](**params)

    def known(self):
        return sorted(self._items)


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block arrangement")
HOOKS = Registry("hook")
FAMILIES = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS}
