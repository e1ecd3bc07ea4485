"""SiLU-gated feed-forward: down( silu(gate(x)) * up(x) ), the residual added in the last
product's epilogue.  gate and up are one stacked product whose rows are [gate | up]
(kernels/fused_silu_fp8_quant.cu:52-56 and v3/crates/rvllm-runtime/src/layer_exec.rs:476-522
of the reference)."""
from __future__ import annotations

from .base import FEED_FORWARDS, Part
from .linear import Linear


class GatedMLP(Part):
    takes_input_norm = True           # the gate/up product can apply the layer's RMSNorm itself

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu"):
        from ..errors import ConfigError
        if activation != "silu":
            raise ConfigError(f"gated MLP activation {activation!r} is not supported (known: silu)")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.gate_up = Linear(hidden_size, [intermediate_size, intermediate_size], ["gate_proj", "up_proj"])
        self.down = Linear(intermediate_size, [hidden_size], ["down_proj"])

    def tensor_specs(self):
        return {**self.gate_up.tensor_specs(), **self.down.tensor_specs()}

    def bind(self, get):
        self.gate_up.bind(get)
        self.down.bind(get)

    def __call__(self, x, ctx, residual=None, input_norm=None):
        h = ctx.kernels.gate_up_silu(x, self.gate_up.weight, norm=input_norm)
        return self.down(h, ctx, residual=residual)


FEED_FORWARDS.register("gated_mlp", GatedMLP)
