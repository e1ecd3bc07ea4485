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
    """A part chosen from a registry (`kind`) with its parameters.  `family` names the registry
    ("mixer", "feed_forward", "norm") where the place of the part does not say it already, as
    among the named parts of a layer."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    family: str = ""


def mixer(kind: str, **params) -> PartSpec:
    return PartSpec(kind, params, "mixer")


def feed_forward(kind: str, **params) -> PartSpec:
    return PartSpec(kind, params, "feed_forward")


def norm(kind: str, **params) -> PartSpec:
    return PartSpec(kind, params, "norm")


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement and the named parts it arranges.

    `parts` maps a role name, which the block arrangement interprets ("mixer", "feed_forward",
    "mixer_norm", "feed_forward_norm" for the pre-norm residual block; a block with four norms,
    or without a feed-forward, has other names), to a part with its family.  At most one part of
    a layer is a mixer: a run entry gives the layer one cache slot.
    `prefix` is the tensor-name prefix of the layer in the checkpoint ("model.layers.3.");
    `names` maps a role to its sub-prefix below that ("self_attn.", "mlp.", ...; default: the
    role name and a dot).
    """
    prefix: str
    block: PartSpec
    parts: Dict[str, PartSpec] = field(default_factory=dict)
    names: Dict[str, str] = field(default_factory=dict)

    @staticmethod
    def standard(prefix: str, block: PartSpec, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec,
                 feed_forward_norm: PartSpec, names: Optional[Dict[str, str]] = None) -> "LayerSpec":
        """The usual four parts: a mixer and a feed-forward, each with the norm in front of it."""
        fam = lambda p, f: PartSpec(p.kind, p.params, p.family or f)
        return LayerSpec(prefix, block, {"mixer": fam(mixer, "mixer"), "feed_forward": fam(feed_forward, "feed_forward"),
                                         "mixer_norm": fam(mixer_norm, "norm"),
                                         "feed_forward_norm": fam(feed_forward_norm, "norm")}, dict(names or {}))


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
    # hooks (registry HOOKS, `__call__(x, ctx) -> x`): on the embedded tokens before the first layer
    # (an embedding scale, ...) and on the float32 logits (a scale, a soft cap, ...), in order
    embedding_hooks: Tuple[PartSpec, ...] = ()
    logit_hooks: Tuple[PartSpec, ...] = ()
    ignored_tensors: Tuple[str, ...] = ()  # fnmatch patterns of checkpoint tensors to skip
    eos_token_ids: Tuple[int, ...] = ()

    def validate(self) -> List[str]:
        problems = []
        for i, layer in enumerate(self.layers):
            for role, part in layer.parts.items():
                if part.family not in ("mixer", "feed_forward", "norm"):
                    problems.append(f"layer {i}: part {role!r} has family {part.family!r} (known: mixer, feed_forward, norm)")
            if sum(1 for part in layer.parts.values() if part.family == "mixer") > 1:
                problems.append(f"layer {i} has more than one mixer; a run entry gives a layer one cache slot")
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
