"""Arrangements of a layer's parts.

`prenorm_residual`: x + mixer(norm(x)), then + feed_forward(norm(.)); the additions happen in
the epilogue of each part's last product (v3/crates/rvllm-runtime/src/layer_exec.rs:189-205,
431-444, 460-474, 511-522 of the reference)."""
from __future__ import annotations

from .base import BLOCKS


class PreNormResidualBlock:
    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm

    def __call__(self, x, ctx, cache, write_cache=True):
        h = self.mixer_norm(x, ctx)
        x = self.mixer(h, ctx, cache, residual=x, write_cache=write_cache)
        h = self.feed_forward_norm(x, ctx)
        return self.feed_forward(h, ctx, residual=x)


BLOCKS.register("prenorm_residual", PreNormResidualBlock)
