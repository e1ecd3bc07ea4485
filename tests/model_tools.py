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


def plain_logits(folder: str, requests: Dict[str, List[int]], device: str = "cpu", rounded: bool = False):
    """float64 logits of the plain implementation, as CPU tensors.  `device`: where its float64
    arithmetic runs (models of real layer widths take minutes on the CPU).  `rounded`: also
    return the logits it gives when every stored activation is rounded to bfloat16."""
    cfg, w = plain_impl.read_model_folder(folder, device=device)
    exact = {rid: plain_impl.forward(cfg, w, toks).cpu() for rid, toks in requests.items()}
    if not rounded:
        return exact
    return exact, {rid: plain_impl.forward(cfg, w, toks, store=plain_impl.round_to_bfloat16).cpu()
                   for rid, toks in requests.items()}


def folder_for(config: dict, seed: int = 0, dtype: str = "bfloat16") -> str:
    """A model folder for any configuration dictionary, written with the framework's
    random-weights mode into a temporary folder."""
    import rvllm_b200
    cfg = rvllm_b200.config_from_dict(config)
    d = tempfile.TemporaryDirectory(prefix="rvllm_cfg_")
    _keep.append(d)
    rvllm_b200.write_random_model(cfg, d.name, seed=seed, dtype=dtype)
    return d.name
