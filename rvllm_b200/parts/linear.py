"""A linear layer y = x W^T (+ b) with W stored [out, in] as in the checkpoints."""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from .base import Part, TensorSpec


class Linear(Part):
    """One matrix, or several matrices with the same input stacked along the output
    dimension (q, k, v; gate, up): the stacked product is one GEMM
    (fusing after v3/crates/rvllm-loader/src/load_multiformat.rs:372-407, 445-477)."""

    def __init__(self, in_features: int, out_features: Sequence[int], names: Sequence[str], bias: bool = False):
        assert len(out_features) == len(names)
        self.in_features = in_features
        self.out_features = list(out_features)
        self.names = list(names)
        self.has_bias = bias
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = {}
        for name, n in zip(self.names, self.out_features):
            specs[f"{name}.weight"] = TensorSpec((n, self.in_features), "matrix")
            if self.has_bias:
                specs[f"{name}.bias"] = TensorSpec((n,), "bias")
        return specs

    def bind(self, get) -> None:
        ws = [get(f"{n}.weight") for n in self.names]
        # matrices stored in different precisions are brought to the widest one
        dt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.weight = (ws[0].to(dt) if len(ws) == 1 else torch.cat([w.to(dt) for w in ws], dim=0)).contiguous()
        if self.has_bias:
            bs = [get(f"{n}.bias") for n in self.names]
            bdt = torch.float32 if any(b.dtype == torch.float32 for b in bs) else bs[0].dtype
            self.bias = (bs[0].to(bdt) if len(bs) == 1 else torch.cat([b.to(bdt) for b in bs], dim=0)).contiguous()

    def __call__(self, x, ctx, residual=None, out_dtype=None, with_bias=True, rows: Optional[int] = None):
        """`rows` limits the product to the first `rows` output features (a leading sub-matrix)."""
        w = self.weight if rows is None else self.weight[:rows]
        b = self.bias if (with_bias and self.bias is not None) else None
        if b is not None and rows is not None:
            b = b[:rows]
        return ctx.kernels.linear(x, w, b, residual, out_dtype)
