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
from .scheduler import PENDING, Request, ScheduledBatch, Scheduler
from .step import StepEntry


@dataclass
class _Flight:
    """A step that has been launched: its batch, the row of each sampling request among the sampled
    ids, the ids on the device, their pinned copy on the host and the event that says it is there."""
    batch: ScheduledBatch
    row_of: Dict[Hashable, int]
    ids: Optional[torch.Tensor] = None
    host_ids: Optional[torch.Tensor] = None
    ready: Optional[object] = None
    host_status: Optional[torch.Tensor] = None      # the kernels' status word, copied with the ids


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
                 enforce_eager: bool = False, async_scheduling: bool = True):
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
        self.async_scheduling = async_scheduling
        self._in_flight: Optional[_Flight] = None
        self._id_buffers: List[Optional[torch.Tensor]] = [None, None]
        self._id_next = 0
        if model is not None:
            from ..tokenizer import Tokenizer
            self.tokenizer = Tokenizer.from_model_dir(model, required=False)

    def capture_graphs(self, max_context: Optional[int] = None) -> int:
        """Capture the CUDA graphs of the decode steps now (every batch bucket, contexts up to
        `max_context`, default max_model_len) instead of at the first step that needs each."""
        return self.engine.runner.capture_decode_graphs(max_context)

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
        """One scheduling decision and one model step; returns the requests that finished.

        With `async_scheduling` a pure decode step is followed at once by the launch of the next
        one, whose tokens are taken from this step's sampled ids on the device; only then does the
        host wait for these ids.  So the device does not idle while the host schedules and packs.
        The tokens produced are the same either way; a request that stops on a token while a step
        ahead of it is running has that step's row ignored."""
        flight = self._in_flight or self._launch(None)
        self._in_flight = None
        if self.async_scheduling and flight.batch.is_decode_only and self.scheduler.can_run_ahead():
            self._in_flight = self._launch(flight)
        finished = self._collect(flight)
        if self._in_flight is not None and all(e.request.state == "finished" for e in self._in_flight.batch.entries):
            self._in_flight = None            # every request of the step ahead stopped: nothing to read from it
        return finished

    def _launch(self, previous: Optional["_Flight"]) -> "_Flight":
        """Schedule, run and sample one step without waiting for the device."""
        batch = self.scheduler.schedule()
        entries, late = [], []
        source = previous.row_of if previous is not None else {}
        for e in batch.entries:
            req = e.request
            toks = req.tokens(e.start, e.num_tokens)
            if toks[-1] == PENDING:           # sampled by the previous step, not read yet
                late.append(source[req.req_id])
                toks = [0]
            else:
                late.append(-1)
            entries.append(StepEntry(req.req_id, toks, (e.num_tokens - 1,) if e.samples else ()))
        late_tokens = (previous.ids, late) if previous is not None and previous.ids is not None else None
        logits = self.engine.runner.step(entries, late_tokens=late_tokens)
        rows = [e.request for e in batch.entries if e.samples]
        flight = _Flight(batch, {r.req_id: i for i, r in enumerate(rows)})
        if rows:
            flight.ids = self.sampler.sample(logits, [r.params for r in rows], [r.seed for r in rows],
                                             [len(r.output) for r in rows])
            if flight.ids.is_cuda:
                host = self._id_buffers[self._id_next]
                self._id_next ^= 1
                if host is None or host.numel() < len(rows) + 1:
                    host = torch.empty((max(len(rows), self.config.max_num_seqs) + 1,), dtype=torch.int32, pin_memory=True)
                    self._id_buffers[self._id_next ^ 1] = host
                flight.host_ids = host[:len(rows)]
                flight.host_ids.copy_(flight.ids, non_blocking=True)
                status = getattr(self.engine.kernels, "status_word", None)
                if status is not None:        # the last element carries the kernels' status word of this step
                    flight.host_status = host[-1:]
                    flight.host_status.copy_(status, non_blocking=True)
                flight.ready = torch.cuda.Event()
                flight.ready.record()
            else:
                flight.host_ids = flight.ids
        self.scheduler.advance(batch)
        return flight

    def _collect(self, flight: "_Flight") -> List[Request]:
        """Wait for the step's sampled ids and account them."""
        sampled: Dict[Hashable, int] = {}
        if flight.host_ids is not None:
            if flight.ready is not None:
                flight.ready.synchronize()
            if flight.host_status is not None and int(flight.host_status[0]) != 0:
                # a kernel of this step gave up a bounded wait: its ids are not results
                self.engine.kernels.raise_on_abort(int(flight.host_status[0]))
            ids = flight.host_ids.tolist()
            sampled = {rid: ids[i] for rid, i in flight.row_of.items()}
        return self.scheduler.resolve(flight.batch, sampled)

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
