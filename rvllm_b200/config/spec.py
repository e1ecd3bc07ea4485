"""The architecture-neutral description a model is built from.

A configuration class (one per architecture) turns its config.json into a `ModelSpec`:
a list of layers, each naming its parts by registry key with their sizes and constants
as parameters, and a run order.  Nothing below this level knows an architecture's name.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """A part chosen from a registry (`kind`) with its parameters."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: which block arrangement, mixer, feed-forward and norms it is made of.

    `prefix` is the tensor-name prefix of the layer in the checkpoint ("model.layers.3.");
    `names` maps each part to its sub-prefix below that ("self_attn.", "mlp.", ...).
    """
    prefix: str
    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    names: Dict[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class RunEntry:
    """One entry of the run order.

    `layer` indexes `ModelSpec.layers` (a layer may appear more than once);
    `cache` is the cache slot the mixer uses: entries with the same number share keys
    and values (or state); `writes_cache` is False for an entry that only reads what
    another entry wrote.
    """
    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_position_embeddings: int
    embedding_name: str
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[RunEntry, ...]
    final_norm: PartSpec
    final_norm_prefix: str
    lm_head_name: Optional[str]          # None: the embedding matrix is the LM head (tied)
    position_encodings: Dict[str, PartSpec] = field(default_factory=dict)
    ignored_tensors: Tuple[str, ...] = ()  # fnmatch patterns of checkpoint tensors to skip
    eos_token_ids: Tuple[int, ...] = ()

    def validate(self) -> List[str]:
        problems = []
        n_cache = {}
        for i, e in enumerate(self.run_order):
            if not 0 <= e.layer < len(self.layers):
                problems.append(f"run_order[{i}] names layer {e.layer}, but there are {len(self.layers)}")
                continue
            owner = n_cache.setdefault(e.cache, None)
            if e.writes_cache:
                if owner is not None:
                    problems.append(f"run_order[{i}]: cache slot {e.cache} is written twice")
                n_cache[e.cache] = i
            elif owner is None:
                problems.append(f"run_order[{i}] reads cache slot {e.cache} before any entry wrote it")
        return problems


def default_run_order(num_layers: int) -> Tuple[RunEntry, ...]:
    """Every layer once, in order, each with a cache slot of its own."""
    return tuple(RunEntry(layer=i, cache=i) for i in range(num_layers))
