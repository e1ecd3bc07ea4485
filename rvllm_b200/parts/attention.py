"""Grouped-query attention over the paged cache.

One step of the mixer (order as v3/crates/rvllm-runtime/src/layer_exec.rs:236-444 of the
reference): fused q/k/v product; bias, rotation of q and k and the write of k and v into the
request's pages in one kernel; attention of the step's tokens over the pages (keys of this
step included, causal, optionally within a window); output product with the residual added in
its epilogue.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import MIXERS, KvCacheNeed, Part
from .linear import Linear


class PagedAttention(Part):
    takes_input_norm = True           # the q/k/v product can apply the layer's input RMSNorm itself

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                 qkv_bias: bool = False, out_bias: bool = False, window: Optional[int] = None,
                 position=None):
        from ..errors import ConfigError
        if num_heads % num_kv_heads:
            raise ConfigError(f"{num_heads} query heads cannot share {num_kv_heads} key/value heads")
        if head_dim % 2 or head_dim > 256:
            raise ConfigError(f"head_dim must be even and at most 256, got {head_dim}")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self.scale, self.window = scale, window
        self.position = position          # a position-encoding part, or None
        q_dim, kv_dim = num_heads * head_dim, num_kv_heads * head_dim
        self.q_dim = q_dim
        self.qkv = Linear(hidden_size, [q_dim, kv_dim, kv_dim], ["q_proj", "k_proj", "v_proj"], bias=qkv_bias)
        self.out = Linear(q_dim, [hidden_size], ["o_proj"], bias=out_bias)

    def tensor_specs(self):
        return {**self.qkv.tensor_specs(), **self.out.tensor_specs()}

    def bind(self, get):
        self.qkv.bind(get)
        self.out.bind(get)

    def cache_need(self):
        return KvCacheNeed(self.num_kv_heads, self.head_dim, self.window)

    def __call__(self, x, ctx, cache, residual=None, write_cache=True, input_norm=None):
        k = ctx.kernels
        meta = ctx.attention[cache.group]
        tables = self.position.rotation_tables() if self.position is not None else None
        cos, sin = tables if tables is not None else (None, None)
        # the bias is added inside the rotation kernel, in float, before the rotation
        bias = self.qkv.bias
        if write_cache:
            q = k.qkv_rope_cache_write(x, self.qkv.weight, bias, ctx.positions, cos, sin, meta.slot_mapping,
                                       cache.kv, self.num_heads, self.num_kv_heads, self.head_dim, norm=input_norm)
        else:                             # a layer that reads another layer's cache needs its queries only
            if input_norm is not None:
                x = k.rmsnorm(x, *input_norm)
            q_rows = self.qkv(x, ctx, with_bias=False, rows=self.q_dim, out_dtype=torch.float32)   # rounded once, after the rotation
            q = k.rope_cache_write(q_rows, bias[:self.q_dim] if bias is not None else None, ctx.positions, cos, sin,
                                   meta.slot_mapping, cache.kv, self.num_heads, self.num_kv_heads, self.head_dim,
                                   write_kv=False, out_dtype=x.dtype)
        o = k.paged_attention(q, cache.kv, meta, self.num_heads, self.num_kv_heads, self.head_dim,
                              self.scale, self.window)
        return self.out(o, ctx, residual=residual)


MIXERS.register("paged_attention", PagedAttention)
