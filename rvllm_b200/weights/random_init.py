"""Random-weights mode: write a model folder (config.json, model.safetensors) from a
configuration and a seed.

Distributions: matrices N(0, 0.02), norm weights 1 + N(0, 0.1), biases N(0, 0.02).  The
reference has no such mode (its benchmarks run on uninitialised caches,
v3/crates/rvllm-runtime/src/bring_up.rs:395-404); these are the distributions this
project's benchmark configurations name.  Tensors are drawn in sorted name order from one
seeded CPU generator, so a (configuration, seed) pair always gives the same file.
"""
from __future__ import annotations

import json
import os
from typing import Dict

import torch

from .safetensors_io import write_safetensors

INIT_STD = {"matrix": (0.0, 0.02), "norm": (1.0, 0.1), "bias": (0.0, 0.02)}


def random_tensors(tensor_specs: Dict[str, "TensorSpec"], seed: int, dtype: torch.dtype,
                   device="cpu") -> Dict[str, torch.Tensor]:
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    out = {}
    for name in sorted(tensor_specs):
        spec = tensor_specs[name]
        mean, std = INIT_STD[spec.init]
        t = torch.empty(spec.shape, dtype=torch.float32, device=device).normal_(mean, std, generator=gen)
        out[name] = t.to(dtype)
    return out


def write_random_model(config, out_dir: str, seed: int = 0, dtype: str = "bfloat16") -> str:
    """Write `out_dir/config.json` and `out_dir/model.safetensors` for `config`
    (any registered configuration object with `to_dict()` and `to_spec()`)."""
    from ..models.decoder import expected_tensors
    os.makedirs(out_dir, exist_ok=True)
    torch_dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    specs = expected_tensors(config.to_spec())
    tensors = random_tensors(specs, seed, torch_dtype)
    cfg = config.to_dict()
    cfg["torch_dtype"] = dtype
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    return out_dir
