"""Continuous batching above the step function.

The reference's scheduler is a skeleton: a step is either one prefill of every queued prompt
whole or one decode of every running request, with no token budget, no page accounting and no
stop on EOS (v3/crates/rvllm-runtime/src/scheduler.rs:37-128, sched_state.rs:9-54); its spec
adds one chunk per step and watermark pre-emption (v3/specs/07-scheduler.md:37-41,74-78).
This scheduler does what the spec sketches:

* every step, running requests go first (oldest first): a decoding request brings one token, a
  partly prefilled one its next portion; then waiting requests are admitted in arrival order
  while request slots, the token budget (`max_num_batched_tokens`) and free pages last;
* a prompt's portion is min(what is left, the budget left, `max_prefill_chunk`); with
  chunking off a prompt is admitted only whole;
* when a running request needs a page and none is free, the most recently admitted running
  request is pre-empted: its pages are given back, it returns to the front of the waiting
  queue and is computed again from its first token (prompt and the tokens it has produced)
  when pages allow - its sampled tokens are kept, so its output does not change;
* a request that could never fit (its prompt plus `max_tokens` need more pages than exist) is
  refused when it is added, with `KvExhausted`;
* a request finishes when it has produced `max_tokens` ("length"), a stop or EOS token
  ("stop"), or has reached `max_model_len` ("length"); its pages and slot are freed at once.

Same arrivals and seeds give the same sequence of batches.

Accounting a step has two halves, so that the next step can be decided while the device still
computes: `advance` counts the step's tokens and appends a stand-in (`PENDING`) for each token
that is being sampled, `resolve` puts the sampled ids in their places and finishes requests.
Between the two, `schedule` treats a stand-in as a token like any other (the step function takes
its value from the device); a request whose pending token is certainly its last is left out.
A request that stops on a token while a later step already runs for it is finished at that
token: the later step's row is ignored and the pages go back at once, which is safe because the
device runs steps in order.  `update` is the two halves together.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence, Tuple

from ..cache import CacheManager
from ..errors import KvExhausted, SchedulerError
from ..sampling.params import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"
PENDING = -1        # stands in `Request.output` for a token that is being sampled


@dataclass(eq=False)        # requests are compared by identity (field-wise equality would walk the token lists)
class Request:
    req_id: Hashable
    prompt: List[int]
    params: SamplingParams
    seed: int = 0
    output: List[int] = field(default_factory=list)
    num_computed: int = 0          # tokens of prompt + output that are in the cache
    state: str = WAITING
    finish_reason: Optional[str] = None
    arrival: int = 0
    num_preemptions: int = 0
    unresolved: int = 0            # stand-ins at the end of `output`

    @property
    def all_tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def remaining(self) -> int:
        return len(self.prompt) + len(self.output) - self.num_computed

    def tokens(self, start: int, n: int) -> List[int]:
        """Tokens [start, start + n) of prompt + output, without joining the two lists."""
        p = len(self.prompt)
        if start >= p:
            return self.output[start - p:start - p + n]
        if start + n <= p:
            return self.prompt[start:start + n]
        return self.prompt[start:] + self.output[:start + n - p]


@dataclass
class ScheduledEntry:
    request: Request
    start: int                     # index of the first token of the portion in prompt + output
    num_tokens: int
    samples: bool                  # True when the portion ends the known tokens: its last row is sampled
    out_index: int = -1            # where in the request's output the sampled token goes (set by advance)


@dataclass
class ScheduledBatch:
    entries: List[ScheduledEntry]
    preempted: List[Request]

    @property
    def num_tokens(self) -> int:
        return sum(e.num_tokens for e in self.entries)

    @property
    def is_decode_only(self) -> bool:
        return bool(self.entries) and all(e.num_tokens == 1 and e.samples for e in self.entries)


class Scheduler:
    def __init__(self, cache: CacheManager, max_num_seqs: int, max_num_batched_tokens: int,
                 max_model_len: int, max_prefill_chunk: Optional[int] = None,
                 enable_chunked_prefill: bool = True, eos_token_ids: Sequence[int] = ()):
        self.cache = cache
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.max_model_len = max_model_len
        self.max_prefill_chunk = max_prefill_chunk
        self.enable_chunked_prefill = enable_chunked_prefill
        self.eos_token_ids = tuple(eos_token_ids)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self._arrivals = 0

    # ---- admission ---------------------------------------------------------------------------
    def add_request(self, req: Request) -> None:
        if not req.prompt:
            raise SchedulerError(f"request {req.req_id!r} has an empty prompt")
        if len(req.prompt) >= self.max_model_len:
            raise SchedulerError(f"request {req.req_id!r}: a prompt of {len(req.prompt)} tokens leaves no room "
                                 f"under max_model_len {self.max_model_len}")
        if not self.enable_chunked_prefill and len(req.prompt) > self.max_num_batched_tokens:
            raise SchedulerError(f"request {req.req_id!r}: a prompt of {len(req.prompt)} tokens exceeds "
                                 f"max_num_batched_tokens {self.max_num_batched_tokens} and chunking is off")
        longest = min(len(req.prompt) + req.params.max_tokens, self.max_model_len)
        # the most pages it will hold at once, group by group: all its tokens where every key is
        # kept, a window plus one step's portion where pages are given back behind the window
        portion = len(req.prompt)
        if self.enable_chunked_prefill:
            portion = min(portion, self.max_num_batched_tokens, self.max_prefill_chunk or portion)
        for gi, need in enumerate(self.cache.peak_pages(longest, portion)):
            if need > self.cache.num_pages:
                raise KvExhausted(need, self.cache.num_pages, f"request {req.req_id!r} can never fit: {longest} tokens "
                                  f"need {need} pages of {self.cache.page_size} at once in cache group {gi}")
        req.arrival = self._arrivals
        self._arrivals += 1
        req.state = WAITING
        self.waiting.append(req)

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- one scheduling decision --------------------------------------------------------------
    def _portion(self, req: Request, budget: int) -> int:
        n = min(req.remaining, budget)
        if req.remaining > 1 and self.max_prefill_chunk is not None:
            n = min(n, self.max_prefill_chunk)
        return n

    def _preempt(self, req: Request, preempted: List[Request]) -> None:
        self.cache.free(req.req_id)
        self.running.remove(req)
        req.num_computed = 0
        req.state = WAITING
        req.num_preemptions += 1
        self.waiting.appendleft(req)
        preempted.append(req)

    def schedule(self) -> ScheduledBatch:
        budget = self.max_num_batched_tokens
        entries: List[ScheduledEntry] = []
        preempted: List[Request] = []
        reserved = [0] * len(self.cache.groups)

        # running requests: decoding ones first, then partly prefilled ones, each oldest first
        order = sorted(self.running, key=lambda r: (r.remaining > 1, r.arrival))
        scheduled_ids = set()
        for req in order:
            if req not in self.running or budget <= 0:
                continue
            if req.unresolved and self._ends_by_length(req):
                continue                    # its pending token is its last
            n = self._portion(req, budget)
            while not self.cache.can_append(req.req_id, n, reserved):
                victim = max((r for r in self.running if r.req_id not in scheduled_ids),
                             key=lambda r: r.arrival, default=None)
                if victim is None:
                    break
                self._preempt(victim, preempted)
                if victim is req:
                    break
            if req not in self.running or not self.cache.can_append(req.req_id, n, reserved):
                continue
            need = self.cache.pages_needed(req.req_id, n)
            reserved = [a + b for a, b in zip(reserved, need)]
            entries.append(ScheduledEntry(req, req.num_computed, n, n == req.remaining))
            scheduled_ids.add(req.req_id)
            budget -= n

        # admissions, in arrival order (pre-empted requests wait at the front)
        while self.waiting and budget > 0 and len(self.running) < self.max_num_seqs:
            req = self.waiting[0]
            if req in preempted:
                break                       # do not re-admit in the step that evicted it
            n = self._portion(req, budget)
            if not self.enable_chunked_prefill and n < req.remaining:
                break
            if not self.cache.can_append(None, n, reserved):
                break
            self.waiting.popleft()
            self.cache.admit(req.req_id)
            req.state = RUNNING
            self.running.append(req)
            need = self.cache.pages_needed(req.req_id, n)
            reserved = [a + b for a, b in zip(reserved, need)]
            entries.append(ScheduledEntry(req, 0, n, n == req.remaining))
            scheduled_ids.add(req.req_id)
            budget -= n

        if not entries and self.has_unfinished():
            # nothing runs and the head of the queue cannot start: it never will
            head = self.waiting[0] if self.waiting else self.running[0]
            need = self.cache.blocks_for(min(head.remaining, self.max_num_batched_tokens))
            raise KvExhausted(need, min(self.cache.num_free_pages() or [0]),
                              f"request {head.req_id!r} cannot be scheduled and nothing is running")
        return ScheduledBatch(entries, preempted)

    # ---- after the step ------------------------------------------------------------------------
    def _ends_by_length(self, req: Request) -> bool:
        return (len(req.output) >= req.params.max_tokens
                or len(req.prompt) + len(req.output) >= self.max_model_len)

    def advance(self, batch: ScheduledBatch) -> None:
        """First half of the accounting, right after the step is launched: its tokens count as
        computed and every token being sampled gets a stand-in in its request's output."""
        for e in batch.entries:
            req = e.request
            req.num_computed += e.num_tokens
            if e.samples:
                e.out_index = len(req.output)
                req.output.append(PENDING)
                req.unresolved += 1

    def resolve(self, batch: ScheduledBatch, sampled: Dict[Hashable, int]) -> List[Request]:
        """Second half: the sampled ids replace their stand-ins; returns the requests that finished.
        Rows of requests that finished at an earlier token are ignored."""
        finished = []
        for e in batch.entries:
            req = e.request
            if not e.samples or req.state == FINISHED:
                continue
            tok = int(sampled[req.req_id])
            req.output[e.out_index] = tok
            req.unresolved -= 1
            reason = None
            stops = set(req.params.stop_token_ids)
            if not req.params.ignore_eos:
                stops.update(self.eos_token_ids)
            if tok in stops:
                reason = "stop"
            elif e.out_index + 1 >= req.params.max_tokens:
                reason = "length"
            elif len(req.prompt) + e.out_index + 1 >= self.max_model_len:
                reason = "length"
            if reason is not None:
                del req.output[e.out_index + 1:]       # stand-ins of steps launched ahead
                req.unresolved = 0
                req.state, req.finish_reason = FINISHED, reason
                if req in self.running:
                    self.running.remove(req)
                else:
                    self.waiting.remove(req)           # pre-empted while its token was pending
                if self.cache.has(req.req_id):
                    self.cache.free(req.req_id)
                finished.append(req)
        return finished

    def can_run_ahead(self) -> bool:
        """True when the next decision is certain before the pending tokens are known: every
        running request decodes, none can be admitted, at least one goes on after its pending
        token, and every one that goes on finds room for one more token."""
        if not self.running or (self.waiting and len(self.running) < self.max_num_seqs):
            return False
        reserved = [0] * len(self.cache.groups)
        goes_on = 0
        for req in self.running:
            if req.remaining != 1:
                return False
            if req.unresolved and self._ends_by_length(req):
                continue
            if not self.cache.can_append(req.req_id, 1, reserved):
                return False
            need = self.cache.pages_needed(req.req_id, 1)
            reserved = [a + b for a, b in zip(reserved, need)]
            goes_on += 1
        return goes_on > 0

    def update(self, batch: ScheduledBatch, sampled: Dict[Hashable, int]) -> List[Request]:
        """Account the step's tokens and the tokens sampled at the ends of portions; returns the
        requests that finished."""
        self.advance(batch)
        return self.resolve(batch, sampled)

    def abort(self, req_id: Hashable) -> None:
        for req in list(self.running):
            if req.req_id == req_id:
                self.running.remove(req)
                self.cache.free(req_id)
                req.state, req.finish_reason = FINISHED, "abort"
        for req in list(self.waiting):
            if req.req_id == req_id:
                self.waiting.remove(req)
                req.state, req.finish_reason = FINISHED, "abort"
