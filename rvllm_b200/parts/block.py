"""Arrangements of a layer's parts.

`prenorm_residual`: x + mixer(norm(x)), then + feed_forward(norm(.)); the additions happen in
the epilogue of each part's last product (v3/crates/rvllm-runtime/src/layer_exec.rs:189-205,
431-444, 460-474, 511-522 of the reference).

A mixer or feed-forward whose class sets `takes_input_norm = True` accepts `input_norm=(gamma,
eps)` and applies that RMSNorm to its input itself (its first product does it in its kernel for
few rows); the block then hands it the unnormalised x.  A norm offers this through `as_rms()`;
parts and norms without these attributes are combined the plain way."""
from __future__ import annotations

from .base import BLOCKS


class PreNormResidualBlock:
    ROLES = ("mixer", "feed_forward", "mixer_norm", "feed_forward_norm")

    def __init__(self, parts):
        from ..errors import ConfigError
        if sorted(parts) != sorted(self.ROLES):
            raise ConfigError(f"the pre-norm residual block arranges the parts {', '.join(self.ROLES)}; got {', '.join(sorted(parts))}")
        self.mixer, self.feed_forward = parts["mixer"], parts["feed_forward"]
        self.mixer_norm, self.feed_forward_norm = parts["mixer_norm"], parts["feed_forward_norm"]

    @staticmethod
    def _handed_over(part, norm):
        if getattr(part, "takes_input_norm", False) and hasattr(norm, "as_rms"):
            return norm.as_rms()
        return None

    def __call__(self, x, ctx, cache, write_cache=True):
        norm = self._handed_over(self.mixer, self.mixer_norm)
        if norm is not None:
            x = self.mixer(x, ctx, cache, residual=x, write_cache=write_cache, input_norm=norm)
        else:
            x = self.mixer(self.mixer_norm(x, ctx), ctx, cache, residual=x, write_cache=write_cache)
        norm = self._handed_over(self.feed_forward, self.feed_forward_norm)
        if norm is not None:
            return self.feed_forward(x, ctx, residual=x, input_norm=norm)
        return self.feed_forward(self.feed_forward_norm(x, ctx), ctx, residual=x)


BLOCKS.register("prenorm_residual", PreNormResidualBlock)
