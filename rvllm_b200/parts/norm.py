"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * gamma, plain gamma, arithmetic in float.

v3/crates/rvllm-fused/src/reference.rs:12-24 and kernels/fused_rmsnorm_fp8_quant.cu:61-84 of
the reference; eps comes from the configuration (the reference hard-codes 1e-6 in two tails,
v3/crates/rvllm-runtime/src/bring_up.rs:1219 - not followed).
"""
from __future__ import annotations

from .base import NORMS, Part, TensorSpec


class RMSNorm(Part):
    def __init__(self, size: int, eps: float):
        self.size, self.eps = size, eps
        self.weight = None

    def tensor_specs(self):
        return {"weight": TensorSpec((self.size,), "norm")}

    def bind(self, get):
        self.weight = get("weight")

    def __call__(self, x, ctx):
        return ctx.kernels.rmsnorm(x, self.weight, self.eps)

    def as_rms(self):
        """(gamma, eps) for a part that applies this norm to its own input (see parts/block.py)."""
        return self.weight, self.eps


NORMS.register("rmsnorm", RMSNorm)
