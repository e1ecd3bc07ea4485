"""The Python entry point: `LLM(...).generate(prompts, sampling_params)`.

The reference's Python package is named `rvllm` and exposes `Sampler`, `Tokenizer` and
`__version__` (tests/test_rvllm_python.py:1-5 of the reference; pyproject.toml:1-30); its
documentation drives engines through `LLM(...).generate()` (docs/profiling.md:63-69).  Option
names follow its command lines: `max_model_len`, `gpu_memory_utilization`, `max_num_seqs`,
`max_num_batched_tokens`, `max_prefill_chunk`, `dtype` (v3/crates/rvllm-serve/src/lib.rs:47-78,
bench_harness.py:21-30).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Union

import torch

from ..config import EngineConfig
from ..errors import ConfigError
from ..sampling import Sampler, SamplingParams, request_seed
from .core import Engine
from .scheduler import Request, ScheduledBatch, Scheduler
from .step import StepEntry


@dataclass
class CompletionOutput:
    token_ids: List[int]
    finish_reason: Optional[str]
    text: Optional[str] = None


@dataclass
class RequestOutput:
    request_id: Hashable
    prompt_token_ids: List[int]
    outputs: List[CompletionOutput]
    num_preemptions: int = 0


class LLM:
    """Offline generation on one B200.

    model: a folder with config.json and model.safetensors (or shards with their index); or
    pass `config=` (a configuration object) with `random_weights=True` and a `seed`.
    """

    def __init__(self, model: Optional[str] = None, *, config=None, random_weights: bool = False, seed: int = 0,
                 dtype: str = "bfloat16", device: str = "cuda:0", block_size: int = 16,
                 num_blocks: Optional[int] = None, gpu_memory_utilization: float = 0.9,
                 max_model_len: Optional[int] = None, max_num_seqs: int = 64, max_num_batched_tokens: int = 2048,
                 max_prefill_chunk: Optional[int] = None, enable_chunked_prefill: bool = True,
                 enforce_eager: bool = False):
        ec = EngineConfig(dtype=dtype, block_size=block_size, num_blocks=num_blocks,
                          gpu_memory_utilization=gpu_memory_utilization, max_model_len=max_model_len,
                          max_num_seqs=max_num_seqs, max_num_batched_tokens=max_num_batched_tokens,
                          max_prefill_chunk=max_prefill_chunk, enable_chunked_prefill=enable_chunked_prefill,
                          enforce_eager=enforce_eager, seed=seed, device=device)
        self.engine = Engine(model, config=config, engine_config=ec, random_weights=random_weights, seed=seed)
        self.config = self.engine.config
        self.sampler = Sampler(self.engine.kernels)
        self.scheduler = self._new_scheduler()
        self.tokenizer = None
        self._next_id = 0
        if model is not None:
            from ..tokenizer import Tokenizer
            self.tokenizer = Tokenizer.from_model_dir(model, required=False)

    def _new_scheduler(self) -> Scheduler:
        ec = self.config
        return Scheduler(self.engine.cache, ec.max_num_seqs, ec.max_num_batched_tokens, ec.max_model_len,
                         ec.max_prefill_chunk, ec.enable_chunked_prefill, self.engine.spec.eos_token_ids)

    # ---- requests ----------------------------------------------------------------------------
    def add_request(self, prompt_token_ids: Sequence[int], params: SamplingParams,
                    request_id: Optional[Hashable] = None) -> Request:
        rid = request_id if request_id is not None else self._next_id
        number = self._next_id
        self._next_id += 1
        seed = params.seed if params.seed is not None else request_seed(self.config.seed, number)
        req = Request(rid, [int(t) for t in prompt_token_ids], params, seed)
        self.scheduler.add_request(req)
        return req

    def step(self) -> List[Request]:
        """One scheduling decision and one model step; returns the requests that finished."""
        batch = self.scheduler.schedule()
        entries = []
        for e in batch.entries:
            toks = e.request.tokens(e.start, e.num_tokens)
            entries.append(StepEntry(e.request.req_id, toks, (e.num_tokens - 1,) if e.samples else ()))
        logits = self.engine.runner.step(entries)
        sampled: Dict[Hashable, int] = {}
        rows = [e.request for e in batch.entries if e.samples]
        if rows:
            ids = self.sampler.sample(logits, [r.params for r in rows], [r.seed for r in rows],
                                      [len(r.output) for r in rows])
            for r, t in zip(rows, ids.tolist()):
                sampled[r.req_id] = t
        return self.scheduler.update(batch, sampled)

    def generate(self, prompts: Union[Sequence[Sequence[int]], Sequence[str]],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> List[RequestOutput]:
        """Generate for every prompt (lists of token ids, or strings when the model folder has a
        tokenizer); outputs come back in the order of the prompts."""
        if sampling_params is None:
            sampling_params = SamplingParams()
        if isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ConfigError(f"{len(prompts)} prompts but {len(sampling_params)} sampling parameter sets")
        reqs = []
        for p, sp in zip(prompts, sampling_params):
            if isinstance(p, str):
                if self.tokenizer is None:
                    raise ConfigError("string prompts need a tokenizer.json in the model folder; pass token ids instead")
                p = self.tokenizer.encode(p)
            reqs.append(self.add_request(p, sp))
        while self.scheduler.has_unfinished():
            self.step()
        outs = []
        for r in reqs:
            text = self.tokenizer.decode(r.output) if self.tokenizer is not None else None
            outs.append(RequestOutput(r.req_id, list(r.prompt), [CompletionOutput(list(r.output), r.finish_reason, text)],
                                      r.num_preemptions))
        return outs
