"""The generic decoder: an embedding, a run order over layers built from registered parts, a
final norm and an LM head.  It is built from a `ModelSpec` alone and does not know which
architecture the spec came from.

Skeleton as the reference's whole-model loop (v3/crates/rvllm-runtime/src/bring_up.rs:535-669
and rvllm-bench/src/bin/rvllm_eval.rs:430-546): gather, layers, then for the wanted rows only
final norm and LM head; the LM head is the embedding matrix when the spec names none
(tie, rvllm-loader/src/load.rs:310-311).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.spec import LayerSpec, ModelSpec, PartSpec
from ..errors import ConfigError
from ..parts.base import BLOCKS, FAMILIES, HOOKS, NORMS, POSITION_ENCODINGS, TensorSpec
from ..parts.linear import Linear


class _Layer:
    def __init__(self, spec: LayerSpec, position_encodings: Dict[str, object]):
        self.spec = spec
        self.parts: Dict[str, object] = {}
        self.mixer = None                  # the part that owns the run entry's cache slot, if the layer has one
        for role, ps in spec.parts.items():
            params = dict(ps.params)
            if ps.family == "mixer" and "position" in params:
                key = params["position"]
                if key is not None and key not in position_encodings:
                    raise ConfigError(f"layer {spec.prefix!r} names position encoding {key!r}, which the model does not define")
                params["position"] = position_encodings.get(key) if key is not None else None
            if ps.family not in FAMILIES:
                raise ConfigError(f"layer {spec.prefix!r}: part {role!r} has family {ps.family!r} (known: {', '.join(FAMILIES)})")
            part = FAMILIES[ps.family].build(ps.kind, **params)
            self.parts[role] = part
            if ps.family == "mixer":
                self.mixer = part
        self.block = BLOCKS.build(spec.block.kind, parts=self.parts, **spec.block.params)

    def cache_need(self):
        return self.mixer.cache_need() if self.mixer is not None else None

    def named_parts(self):
        n = self.spec.names
        return [(self.spec.prefix + n.get(role, role + "."), part) for role, part in self.parts.items()]


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        problems = spec.validate()
        if problems:
            raise ConfigError(problems, "model spec")
        self.spec = spec
        self.position_encodings = {k: POSITION_ENCODINGS.build(p.kind, **p.params)
                                   for k, p in spec.position_encodings.items()}
        self.layers: List[_Layer] = [_Layer(ls, self.position_encodings) for ls in spec.layers]
        self.final_norm = NORMS.build(spec.final_norm.kind, **spec.final_norm.params)
        self.embedding_hooks = [HOOKS.build(h.kind, **h.params) for h in spec.embedding_hooks]
        self.logit_hooks = [HOOKS.build(h.kind, **h.params) for h in spec.logit_hooks]
        self.embedding: Optional[torch.Tensor] = None
        self.lm_head: Optional[torch.Tensor] = None
        self.dtype = None
        self.device = None

    # ---- tensors ---------------------------------------------------------------------------
    def named_parts(self):
        out = []
        for layer in self.layers:
            out.extend(layer.named_parts())
        out.append((self.spec.final_norm_prefix, self.final_norm))
        for key, pe in self.position_encodings.items():
            out.append((f"position.{key}.", pe))
        out.extend((f"hooks.embedding.{i}.", h) for i, h in enumerate(self.embedding_hooks))
        out.extend((f"hooks.logits.{i}.", h) for i, h in enumerate(self.logit_hooks))
        return out

    @property
    def graph_safe(self) -> bool:
        """Whether a decode step of this model may be captured in a CUDA graph: every part (and
        block arrangement) allows it."""
        things = [part for _, part in self.named_parts()] + [layer.block for layer in self.layers]
        return all(getattr(t, "graph_safe", True) for t in things)

    def expected_tensors(self) -> Dict[str, TensorSpec]:
        s = self.spec
        specs = {s.embedding_name: TensorSpec((s.vocab_size, s.hidden_size), "matrix")}
        if s.lm_head_name is not None:
            specs[s.lm_head_name] = TensorSpec((s.vocab_size, s.hidden_size), "matrix")
        for prefix, part in self.named_parts():
            for name, ts in part.tensor_specs().items():
                specs[prefix + name] = ts
        return specs

    def load(self, get, dtype: torch.dtype, device, max_len: int) -> None:
        """`get(full tensor name)` -> tensor on `device` in its engine dtype."""
        self.dtype, self.device = dtype, torch.device(device)
        self.embedding = get(self.spec.embedding_name)
        self.lm_head = get(self.spec.lm_head_name) if self.spec.lm_head_name is not None else self.embedding
        for prefix, part in self.named_parts():
            part.bind(lambda name, _p=prefix: get(_p + name))
        for pe in self.position_encodings.values():
            pe.prepare(max_len, device)

    # ---- what the cache manager has to provide ---------------------------------------------------
    def cache_needs(self) -> Dict[int, object]:
        """cache slot -> KvCacheNeed | StateNeed | None, taken from the entry that writes it."""
        needs = {}
        for e in self.spec.run_order:
            need = self.layers[e.layer].cache_need()
            if e.writes_cache:
                needs[e.cache] = need
        for e in self.spec.run_order:
            if not e.writes_cache:
                need = self.layers[e.layer].cache_need()
                if need != needs.get(e.cache):
                    raise ConfigError(f"layer {e.layer} reads cache slot {e.cache} but needs {need}, "
                                      f"while its writer provides {needs.get(e.cache)}")
        return needs

    # ---- the forward pass of one step ----------------------------------------------------------
    def forward(self, ctx, caches) -> torch.Tensor:
        x = ctx.kernels.gather_rows(self.embedding, ctx.token_ids)
        if x.dtype != self.dtype:
            x = x.to(self.dtype)       # a table the checkpoint keeps in 32 bits; activations have the engine's type
        for pe in self.position_encodings.values():
            x = pe.on_embeddings(x, ctx)
        for hook in self.embedding_hooks:
            x = hook(x, ctx)
        for e in self.spec.run_order:
            x = self.layers[e.layer].block(x, ctx, caches.view(e.cache), e.writes_cache)
        return x

    def compute_logits(self, hidden: torch.Tensor, ctx) -> torch.Tensor:
        """float32 logits [R, vocab] at the rows `ctx.logit_rows` of the step."""
        rows = ctx.kernels.gather_rows(hidden, ctx.logit_rows)
        if hasattr(self.final_norm, "as_rms"):       # the LM head's product applies the norm itself for few rows
            logits = ctx.kernels.linear(rows, self.lm_head, None, None, torch.float32, norm=self.final_norm.as_rms())
        else:
            logits = ctx.kernels.linear(self.final_norm(rows, ctx), self.lm_head, None, None, torch.float32)
        for hook in self.logit_hooks:
            logits = hook(logits, ctx)
        return logits


def expected_tensors(spec: ModelSpec) -> Dict[str, TensorSpec]:
    return DecoderModel(spec).expected_tensors()
