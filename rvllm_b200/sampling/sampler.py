"""Sampling of one token per logits row on the device.

`Sampler.sample` gathers the rows' parameters into small tensors, launches the sampling
kernel and returns the token ids; only these ids leave the GPU
(as in the reference, v3/crates/rvllm-runtime/src/bring_up.rs:1443-1454).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..errors import SamplingError
from .params import SamplingParams


def request_seed(engine_seed: int, request_number: int) -> int:
    """Seed of a request that brought none: a fixed mix of the engine's seed and the request's
    arrival number (splitmix64 finaliser), so that runs repeat."""
    z = (engine_seed * 0x9E3779B97F4A7C15 + request_number + 1) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    return (z ^ (z >> 31)) & 0x7FFFFFFFFFFFFFFF


class Sampler:
    def __init__(self, kernels=None, device="cuda:0"):
        if kernels is None:
            from ..kernels import get_library
            kernels = get_library(device)
        self.kernels = kernels

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               draw_index: Sequence[int]) -> torch.Tensor:
        """logits float32 [R, V]; one parameter set, seed and output index per row.
        Returns int32 token ids [R] on the device."""
        R = logits.shape[0]
        if not (len(params) == len(seeds) == len(draw_index) == R):
            raise SamplingError(f"{R} logits rows but {len(params)} parameter sets, {len(seeds)} seeds, "
                                f"{len(draw_index)} draw indices")
        if all(p.is_greedy for p in params):
            return self.kernels.sample(logits)
        dev = logits.device
        host = torch.tensor([[p.temperature, p.top_p] for p in params], dtype=torch.float32)
        ints = torch.tensor([[p.top_k] for p in params], dtype=torch.int32)
        longs = torch.tensor([list(seeds), list(draw_index)], dtype=torch.int64)
        host, ints, longs = host.to(dev, non_blocking=True), ints.to(dev, non_blocking=True), longs.to(dev, non_blocking=True)
        use_k = any(p.top_k > 0 for p in params)
        use_p = any(p.top_p < 1.0 for p in params)
        return self.kernels.sample(logits, host[:, 0].contiguous(), ints[:, 0].contiguous() if use_k else None,
                                   host[:, 1].contiguous() if use_p else None, longs[0], longs[1])
