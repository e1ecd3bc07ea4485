"""Putting the engine together: configuration -> model -> weights -> cache -> step function.

Start-up follows the reference's `Bringup::load` in spirit
(v3/crates/rvllm-runtime/src/bring_up.rs:81-220: configuration, weights fully resident before
the first step, then the caches sized from what memory is left).
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch

from ..cache import CacheManager
from ..config import EngineConfig, load_config
from ..errors import ConfigError, KernelError
from ..kernels import get_library
from ..models import DecoderModel
from ..parts.base import KvCacheNeed
from ..weights import WeightSource
from ..weights.random_init import INIT_STD
from .step import ModelRunner

_TORCH_DTYPE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


class Engine:
    """Model, cache and step function on one device."""

    def __init__(self, model_dir: Optional[str] = None, *, config=None, engine_config: Optional[EngineConfig] = None,
                 random_weights: bool = False, seed: int = 0):
        if (model_dir is None) == (config is None):
            raise ConfigError("give either a model folder or a configuration object (with random_weights=True)")
        if config is None:
            config = load_config(model_dir)
        elif not random_weights:
            raise ConfigError("a configuration without a model folder needs random_weights=True")
        self.model_config = config
        self.spec = config.to_spec()
        ec = (engine_config or EngineConfig()).validated(self.spec.max_position_embeddings)
        self.config = ec
        self.device = torch.device(ec.device)
        self.dtype = _TORCH_DTYPE[ec.dtype]
        self.kernels = get_library(ec.device)
        self.model = DecoderModel(self.spec)

        expected = self.model.expected_tensors()
        if random_weights and model_dir is None:
            if hasattr(self.kernels, "fill_normal"):
                # filled on the device by the counter-based generator: a tensor's values depend on the
                # seed and on its place among the sorted names only
                order = {name: i for i, name in enumerate(sorted(expected))}

                def get(name: str) -> torch.Tensor:
                    ts = expected[name]
                    mean, std = INIT_STD[ts.init]
                    return self.kernels.fill_normal(ts.shape, self.dtype, mean, std, seed, order[name])
            else:
                gen = torch.Generator(device=self.device)
                gen.manual_seed(seed)

                def get(name: str) -> torch.Tensor:
                    ts = expected[name]
                    mean, std = INIT_STD[ts.init]
                    t = torch.empty(ts.shape, dtype=torch.float32, device=self.device).normal_(mean, std, generator=gen)
                    return t.to(self.dtype)
        else:
            source = WeightSource(model_dir)
            source.check({n: ts.shape for n, ts in expected.items()}, self.spec.ignored_tensors)

            def get(name: str) -> torch.Tensor:
                return source.get(name, self.dtype, self.device)
        self.model.load(get, self.dtype, self.device, ec.max_model_len)

        needs = self.model.cache_needs()
        num_pages = ec.num_blocks if ec.num_blocks is not None else self._pages_from_memory(needs, ec)
        self.cache = CacheManager(needs, num_pages, ec.block_size, ec.max_num_seqs, self.dtype, self.device)
        self.runner = ModelRunner(self.model, self.cache, self.kernels, ec.max_model_len, self.device,
                                  () if ec.enforce_eager else ec.cuda_graph_batch_sizes)

    def _pages_from_memory(self, needs: Dict[int, object], ec: EngineConfig) -> int:
        per_page = CacheManager.bytes_per_page(needs, ec.block_size, self.dtype)
        most = ec.max_num_seqs * ((ec.max_model_len + ec.block_size - 1) // ec.block_size)
        if per_page == 0:
            return 1
        if self.device.type != "cuda":
            return min(most, 4096)
        free, total = torch.cuda.mem_get_info(self.device)
        # leave room for the activations of a full step and the logits of its wanted rows
        el = 2 if self.dtype == torch.bfloat16 else 4
        # a step keeps a handful of [tokens, hidden] buffers and two of the widest projection
        act = ec.max_num_batched_tokens * self.spec.hidden_size * el * 24
        act += ec.max_num_seqs * self.spec.vocab_size * 4 * 3
        usable = free - (1.0 - ec.gpu_memory_utilization) * total - act - (1 << 30)
        pages = int(usable // per_page)
        if pages < 1:
            raise ConfigError(f"no memory left for the cache: {free / 2**30:.1f} GiB free, "
                              f"{per_page / 2**20:.2f} MiB per page", "engine options")
        return min(pages, most)
