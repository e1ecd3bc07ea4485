"""Helpers shared by the tests: tiny model folders and plain logits for them."""
from __future__ import annotations

import functools
import tempfile
from typing import Dict, List

import torch

import plain_impl
import tiny_configs

_keep = []   # temporary folders live as long as the test session


@functools.lru_cache(maxsize=None)
def model_folder(name: str, seed: int = 0, dtype: str = "bfloat16") -> str:
    """A model folder for the named tiny configuration, written with the framework's own
    random-weights mode into a temporary folder."""
    import rvllm_b200
    cfg = rvllm_b200.config_from_dict(tiny_configs.get(name))
    d = tempfile.TemporaryDirectory(prefix=f"rvllm_{name}_")
    _keep.append(d)
    rvllm_b200.write_random_model(cfg, d.name, seed=seed, dtype=dtype)
    return d.name


def random_requests(vocab: int, lengths, seed: int = 0) -> Dict[str, List[int]]:
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(lengths)}


def plain_logits(folder: str, requests: Dict[str, List[int]]) -> Dict[str, torch.Tensor]:
    cfg, w = plain_impl.read_model_folder(folder)
    return {rid: plain_impl.forward(cfg, w, toks) for rid, toks in requests.items()}
