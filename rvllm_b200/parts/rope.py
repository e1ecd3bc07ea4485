"""Rotary position encoding: frequency table, optional llama3 scaling, cos/sin tables.

inv_freq_i = theta^(-2i/head_dim) (v3/crates/rvllm-loader/src/load.rs:876-891 of the
reference).  The reference never reads `rope_scaling`; the llama3 rule is the published one:
with wavelength L = 2 pi / inv_freq, L < orig/high keeps the frequency, L > orig/low divides
it by `factor`, and between the two it is blended with s = (orig/L - low) / (high - low).
Frequencies are computed in float64 and kept as float32; angles position * inv_freq and
their cos/sin are computed in float64 and the tables kept as float32 (the reference rounds
them to half precision, which this engine does not).  Pairs are (i, i + head_dim/2)
(v3/crates/rvllm-fused/src/reference.rs:177-203).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..errors import ConfigError
from .base import POSITION_ENCODINGS, Part


def inverse_frequencies(head_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    half = head_dim // 2
    inv = torch.tensor([float(theta) ** (-2.0 * i / head_dim) for i in range(half)], dtype=torch.float64)
    if scaling:
        kind = scaling.get("rope_type", "default")
        if kind == "llama3":
            factor = float(scaling["factor"])
            low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
            orig = float(scaling["original_max_position_embeddings"])
            wavelen = 2.0 * math.pi / inv
            smooth = (orig / wavelen - low) / (high - low)
            blended = (1.0 - smooth) * inv / factor + smooth * inv
            inv = torch.where(wavelen < orig / high, inv, torch.where(wavelen > orig / low, inv / factor, blended))
        elif kind != "default":
            raise ConfigError(f"rotary scaling {kind!r} is not supported (known: default, llama3)")
    return inv.to(torch.float32)


class RotaryEncoding(Part):
    """`rotary_dim` (default: head_dim) is the number of leading elements of a head that are
    rotated, in pairs (i, i + rotary_dim/2) with frequencies theta^(-2i/rotary_dim); the rest of
    the head passes through.  The tables then have rotary_dim/2 columns, and the kernels that
    rotate in a GEMM's epilogue (whole heads only) leave such a model to the rotary kernel."""

    def __init__(self, head_dim: int, theta: float, scaling: Optional[dict] = None, rotary_dim: Optional[int] = None):
        if head_dim % 2:
            raise ConfigError(f"rotary encoding needs an even head_dim, got {head_dim}")
        rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if rotary_dim % 2 or not 0 < rotary_dim <= head_dim:
            raise ConfigError(f"rotary_dim must be even and in (0, head_dim = {head_dim}], got {rotary_dim}")
        self.head_dim, self.theta, self.scaling, self.rotary_dim = head_dim, theta, scaling, rotary_dim
        self.inv_freq = inverse_frequencies(rotary_dim, theta, scaling)
        self.cos = self.sin = None

    def prepare(self, max_len: int, device) -> None:
        cos = torch.empty((max_len, self.rotary_dim // 2), dtype=torch.float32)
        sin = torch.empty_like(cos)
        inv = self.inv_freq.to(torch.float64)
        step = 16384
        for s in range(0, max_len, step):
            pos = torch.arange(s, min(max_len, s + step), dtype=torch.float64)
            ang = pos[:, None] * inv[None, :]
            cos[s:s + step] = torch.cos(ang).to(torch.float32)
            sin[s:s + step] = torch.sin(ang).to(torch.float32)
        self.cos, self.sin = cos.to(device), sin.to(device)

    def rotation_tables(self):
        return self.cos, self.sin

    def on_embeddings(self, x, ctx):
        return x


POSITION_ENCODINGS.register("rotary", RotaryEncoding)
