"""The scheduler's decisions: admission, portions under the token budget, decoding, finishing
and freeing, and what happens when pages run out."""
import pytest
import torch

from rvllm_b200 import KvExhausted, SamplingParams, SchedulerError
from rvllm_b200.cache import CacheManager
from rvllm_b200.engine import Request, Scheduler
from rvllm_b200.parts import KvCacheNeed


def make(num_pages=64, page=4, max_seqs=4, budget=16, chunk=None, chunked=True, max_len=256, eos=()):
    cache = CacheManager({0: KvCacheNeed(1, 16, None)}, num_pages, page, max_seqs, allocate=False)
    return cache, Scheduler(cache, max_seqs, budget, max_len, chunk, chunked, eos)


def run_step(cache, sched, token_of=lambda req: 100 + len(req.output)):
    """Do what the engine does with a batch: reserve the pages, then report sampled tokens."""
    batch = sched.schedule()
    for e in batch.entries:
        cache.append(e.request.req_id, e.num_tokens)
    sampled = {e.request.req_id: token_of(e.request) for e in batch.entries if e.samples}
    finished = sched.update(batch, sampled)
    cache.check()
    return batch, finished


def req(rid, n_prompt, max_tokens=4, **kw):
    return Request(rid, list(range(1, n_prompt + 1)), SamplingParams(max_tokens=max_tokens, **kw))


def test_prompts_are_cut_under_the_token_budget_and_decodes_go_first():
    cache, s = make(budget=16)
    s.add_request(req("a", 20))
    s.add_request(req("b", 5))
    b1, _ = run_step(cache, s)
    assert [(e.request.req_id, e.start, e.num_tokens, e.samples) for e in b1.entries] == [("a", 0, 16, False)]
    b2, _ = run_step(cache, s)
    assert [(e.request.req_id, e.start, e.num_tokens, e.samples) for e in b2.entries] == [("a", 16, 4, True), ("b", 0, 5, True)]
    b3, _ = run_step(cache, s)          # both decode now: one token each
    assert [(e.request.req_id, e.num_tokens) for e in b3.entries] == [("a", 1), ("b", 1)] and b3.is_decode_only
    s.add_request(req("c", 30))
    b4, _ = run_step(cache, s)          # decodes first, the new prompt gets what is left of the budget
    assert [(e.request.req_id, e.num_tokens) for e in b4.entries] == [("a", 1), ("b", 1), ("c", 14)]
    assert b4.num_tokens == 16


def test_max_prefill_chunk_and_unchunked_mode():
    cache, s = make(budget=64, chunk=6)
    s.add_request(req("a", 15))
    sizes = []
    while not s.running or s.running[0].remaining > 1:
        b, _ = run_step(cache, s)
        sizes.append(b.entries[0].num_tokens)
        if b.entries[0].samples:
            break
    assert sizes == [6, 6, 3]
    cache, s = make(budget=16, chunked=False)
    s.add_request(req("a", 10))
    s.add_request(req("b", 10))
    b, _ = run_step(cache, s)           # b would have to be cut: it waits
    assert [e.request.req_id for e in b.entries] == ["a"]
    with pytest.raises(SchedulerError, match="chunking is off"):
        s.add_request(req("c", 17))


def test_finishing_reasons_and_freeing():
    cache, s = make(eos=(7,), max_len=12)
    s.add_request(req("len", 3, max_tokens=2))
    s.add_request(req("eos", 3, max_tokens=50))
    s.add_request(req("stop", 3, max_tokens=50, stop_token_ids=(9,)))
    s.add_request(req("cap", 8, max_tokens=50, ignore_eos=True))
    toks = {"len": [1, 1], "eos": [1, 7], "stop": [1, 1, 9], "cap": [7, 7, 7, 7, 7]}
    done = {}
    for _ in range(8):
        if not s.has_unfinished():
            break
        _, fin = run_step(cache, s, token_of=lambda r: toks[r.req_id][len(r.output)])
        for r in fin:
            done[r.req_id] = (r.finish_reason, list(r.output))
    assert done == {"len": ("length", [1, 1]), "eos": ("stop", [1, 7]), "stop": ("stop", [1, 1, 9]),
                    "cap": ("length", [7, 7, 7, 7])}     # 8 + 4 = max_model_len 12; EOS ignored
    assert cache.num_free_pages() == [64] and cache.slots.num_free == 4 and not cache.requests


def test_admission_is_limited_by_slots_and_pages():
    cache, s = make(num_pages=6, page=4, max_seqs=2, budget=64)
    for i in range(3):
        s.add_request(req(f"r{i}", 8, max_tokens=2))
    b, _ = run_step(cache, s)
    assert [e.request.req_id for e in b.entries] == ["r0", "r1"]          # two slots
    cache, s = make(num_pages=5, page=4, max_seqs=4, budget=64)
    for i in range(3):
        s.add_request(req(f"r{i}", 8, max_tokens=2))
    b, _ = run_step(cache, s)
    assert [e.request.req_id for e in b.entries] == ["r0", "r1"]          # 2 + 2 pages, the third prompt has no room
    with pytest.raises(KvExhausted, match="never fit"):
        s.add_request(req("huge", 8, max_tokens=100))
    with pytest.raises(SchedulerError, match="empty"):
        s.add_request(Request("e", [], SamplingParams()))


def test_running_out_of_pages_preempts_the_newest_and_recomputes_it():
    cache, s = make(num_pages=6, page=4, max_seqs=4, budget=64)
    s.add_request(req("old", 8, max_tokens=12))
    s.add_request(req("new", 8, max_tokens=12))
    outputs = {}
    preempted = []
    steps = 0
    while s.has_unfinished():
        batch, fin = run_step(cache, s)
        preempted += [r.req_id for r in batch.preempted]
        for r in fin:
            outputs[r.req_id] = list(r.output)
        steps += 1
        assert steps < 200
    assert preempted and set(preempted) == {"new"}                        # the oldest request is never evicted
    assert outputs["old"] == [100 + i for i in range(12)]
    assert outputs["new"] == [100 + i for i in range(12)]                 # its sampled tokens were kept
    assert cache.num_free_pages() == [6]


def test_a_preempted_request_is_prefilled_again_with_its_output():
    cache, s = make(num_pages=5, page=4, max_seqs=4, budget=64)
    s.add_request(req("old", 8, max_tokens=9))
    s.add_request(req("new", 7, max_tokens=9))
    seen = []
    while s.has_unfinished():
        batch, _ = run_step(cache, s)
        for e in batch.entries:
            if e.request.req_id == "new":
                seen.append((e.start, e.num_tokens, len(e.request.output)))
    restarts = [x for x in seen[1:] if x[0] == 0]
    assert restarts, "the evicted request starts again at position 0"
    start, n, produced = restarts[0]
    # `produced` was read after the step, which sampled one more token at the portion's end
    assert n == 7 + produced - 1 and produced > 1                         # prompt and what it had produced


def test_nothing_schedulable_is_an_error_not_a_spin():
    cache, s = make(num_pages=4, page=4, max_seqs=4, budget=64)
    cache.admit("squatter")
    cache.append("squatter", 12)                                          # someone else holds 3 of 4 pages
    s.add_request(req("a", 6, max_tokens=2))
    with pytest.raises(KvExhausted, match="cannot be scheduled"):
        s.schedule()


def test_same_arrivals_give_the_same_batches():
    def trace():
        cache, s = make(num_pages=10, page=4, max_seqs=3, budget=12, chunk=5)
        for i, n in enumerate([9, 3, 14, 6, 2]):
            s.add_request(req(f"r{i}", n, max_tokens=5))
        out = []
        while s.has_unfinished():
            b, _ = run_step(cache, s)
            out.append([(e.request.req_id, e.start, e.num_tokens, e.samples) for e in b.entries])
        return out
    assert trace() == trace()


def test_abort_frees():
    cache, s = make()
    s.add_request(req("a", 5))
    s.add_request(req("b", 5))
    run_step(cache, s)
    s.abort("a")
    s.abort("b")
    assert not s.has_unfinished() and cache.num_free_pages() == [64]


def test_two_halves_of_the_accounting_let_a_step_run_ahead():
    """advance / resolve: the next decode step is decided while tokens are pending; a request whose
    pending token is its last is left out; one that stops while a step ahead of it runs is finished
    at the stop token, the row ahead is ignored and its pages go back."""
    from rvllm_b200.engine.scheduler import PENDING
    cache, s = make(budget=16, eos=(7,))
    s.add_request(req("a", 5, max_tokens=3))
    s.add_request(req("b", 6, max_tokens=8))
    s.add_request(req("c", 3, max_tokens=8))
    b0, _ = run_step(cache, s, token_of=lambda r: 50)             # prompts whole, first tokens
    assert not s.can_run_ahead() or b0.is_decode_only is False
    b1 = s.schedule()                                             # step 1: all decode
    for e in b1.entries:
        cache.append(e.request.req_id, 1)
    s.advance(b1)
    a, b, c = (e.request for e in b1.entries)
    assert a.output == [50, PENDING] and a.unresolved == 1 and a.remaining == 1
    assert s.can_run_ahead()
    b2 = s.schedule()                                             # step 2, decided before step 1 is read
    assert [e.request.req_id for e in b2.entries] == ["a", "b", "c"]
    assert [e.request.tokens(e.start, 1) for e in b2.entries] == [[PENDING]] * 3
    for e in b2.entries:
        cache.append(e.request.req_id, 1)
    s.advance(b2)
    assert a.output == [50, PENDING, PENDING]
    assert s.can_run_ahead()                                      # a ends with its pending token, b and c go on
    done = s.resolve(b1, {"a": 51, "b": 7, "c": 52})              # b stops on EOS while step 2 runs for it
    assert [r.req_id for r in done] == ["b"] and b.output == [50, 7] and b.finish_reason == "stop"
    assert not cache.has("b") and b not in s.running
    b3 = s.schedule()                                             # a is not scheduled: its third token is its last
    assert [e.request.req_id for e in b3.entries] == ["c"]
    cache.append("c", 1)
    s.advance(b3)
    done = s.resolve(b2, {"a": 53, "b": 99, "c": 54})             # b's row of the step ahead is ignored
    assert [r.req_id for r in done] == ["a"] and a.output == [50, 51, 53] and a.finish_reason == "length"
    assert b.output == [50, 7] and c.output == [50, 52, 54, PENDING]
    s.resolve(b3, {"c": 7})
    assert c.output == [50, 52, 54, 7] and c.finish_reason == "stop"
    assert not s.has_unfinished() and not cache.requests
    cache.check()
    assert cache.num_free_pages() == [64]


def test_a_window_only_model_admits_requests_longer_than_its_pool():
    """Every group of this cache keeps a window of 16 keys: a request holds the window plus one
    step's portion at most, so a request of 200 tokens fits a pool of 10 pages of 4 - and runs to
    its end with pages coming back behind the window.  With a group that keeps every key beside it
    the same request can never fit, and the error names that group."""
    def run(needs, budget, num_pages=10):
        cache = CacheManager(needs, num_pages, 4, 2, allocate=False)
        s = Scheduler(cache, 2, budget, 256, None, True, ())
        s.add_request(req("long", 150, max_tokens=50))
        peak = 0
        while s.has_unfinished():
            batch = s.schedule()
            assert not batch.preempted
            for e in batch.entries:
                cache.append(e.request.req_id, e.num_tokens)
            peak = max(peak, num_pages - min(cache.num_free_pages()))
            for e in batch.entries:
                cache.release_passed(e.request.req_id)          # as the step function does after the model ran
            s.update(batch, {e.request.req_id: 7 for e in batch.entries if e.samples})
            cache.check()
        return cache, peak
    cache, peak = run({0: KvCacheNeed(1, 16, 16), 1: KvCacheNeed(1, 16, 16)}, budget=8)
    assert cache.peak_pages(200, 8) == [7] and peak <= 7 and cache.num_free_pages() == [10]
    with pytest.raises(KvExhausted, match="never fit.*group 1"):
        run({0: KvCacheNeed(1, 16, 16), 1: KvCacheNeed(1, 16, None)}, budget=8)
    with pytest.raises(KvExhausted, match="never fit.*group 0"):
        run({0: KvCacheNeed(1, 16, 16)}, budget=64)                 # portions of 64 tokens do not fit 10 pages
