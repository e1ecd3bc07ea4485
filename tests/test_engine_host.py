"""The engine's host side without a GPU: the real step function, cache manager, scheduler,
trace replay and entry point, driven with torch stand-ins for the kernels (emulated_kernels.py)
and compared with the plain implementation.  What is checked here is the bookkeeping - paging,
block tables, slot mapping, portions, page reuse, padding; the kernels themselves are checked by
the GPU tests."""
import io
import os

import numpy as np
import pytest
import torch

import plain_impl
import tiny_configs
import trace_tools as TT
from emulated_kernels import EmulatedKernels
from model_tools import model_folder, plain_logits, random_requests

from rvllm_b200 import KernelError, LLM, SamplingParams, kernels as kernel_pkg, load_config
from rvllm_b200.engine import trace as trace_mod


@pytest.fixture
def emulated():
    kernel_pkg.set_library(EmulatedKernels())
    yield
    kernel_pkg.set_library(None)


def test_no_cpu_path_without_injection():
    kernel_pkg.set_library(None)
    with pytest.raises(KernelError, match="CUDA"):
        kernel_pkg.get_library("cpu")


LENGTHS = {"tiny_llama": (45, 70, 33, 81, 100, 38), "tiny_qwen2": (90, 37, 110, 64, 51, 75)}
SCHEDULES = {
    "whole": TT.schedule_whole,
    "bulk_tail": TT.schedule_bulk_tail,
    "portions": TT.schedule_portions,
    "mixed": TT.schedule_mixed,
}


@pytest.mark.parametrize("name", ["tiny_llama", "tiny_qwen2"])
@pytest.mark.parametrize("schedule", list(SCHEDULES))
def test_replay_matches_plain_under_every_cut(emulated, tmp_path, name, schedule):
    folder = model_folder(name)
    vocab = load_config(folder).vocab_size
    reqs = random_requests(vocab, LENGTHS[name], seed=3)
    ref = plain_logits(folder, reqs)
    trace = SCHEDULES[schedule](reqs)
    if schedule == "portions":
        assert min(len(e["tokens"]) for s in trace.steps for e in s["entries"]) <= 2
    if schedule == "mixed":
        assert max(len(s["entries"]) for s in trace.steps) == 4
        assert any(len({len(e["tokens"]) == 1 for e in s["entries"]}) == 2 for s in trace.steps), \
            "portions beside single tokens"
        assert trace.preemptions == 1 and any(label.endswith("#0") for rows in trace.rows.values() for label, _ in rows), \
            "one live request is ended and fed again from position 0"
    engine = trace_mod.build_engine(folder, "float32", trace.max_tokens, block_size=8, device="cpu")
    pages = engine.cache.num_pages
    assert pages * 8 == trace.max_tokens                       # so few pages that they are used again
    echo = io.StringIO()
    n = trace_mod.replay(engine, io.StringIO(trace.lines()), str(tmp_path), echo)
    assert n == len(trace.steps) and echo.getvalue().splitlines() == [f"done {i}" for i in range(n)]
    got = TT.read_logits(str(tmp_path), trace, vocab)
    worst = TT.compare(got, ref, 1e-5, f"{name}/{schedule}")
    engine.cache.check()
    assert engine.cache.num_free_pages() == [pages] * len(engine.cache.groups) and not engine.cache.requests
    assert worst < 1e-5


def test_generate_greedy_matches_plain(emulated):
    folder = model_folder("tiny_llama")
    cfg, w = plain_impl.read_model_folder(folder)
    prompts = list(random_requests(cfg["vocab_size"], (5, 17, 33), seed=9).values())
    llm = LLM(folder, dtype="float32", device="cpu", block_size=16, num_blocks=12, max_model_len=64,
              max_num_seqs=3, max_num_batched_tokens=24, max_prefill_chunk=16)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.outputs[0].token_ids == plain_impl.greedy_generate(cfg, w, p, 8)
        assert o.outputs[0].finish_reason == "length" and o.prompt_token_ids == p
    llm.engine.cache.check()
    assert llm.engine.cache.num_free_pages() == [12]


def test_generate_survives_preemption_with_the_same_tokens(emulated):
    folder = model_folder("tiny_qwen2")
    cfg = load_config(folder)
    prompts = list(random_requests(cfg.vocab_size, (30, 28, 26, 20), seed=4).values())
    sp = SamplingParams(temperature=0.8, seed=123, max_tokens=12, ignore_eos=True)
    roomy = LLM(folder, dtype="float32", device="cpu", block_size=8, num_blocks=64, max_model_len=128,
                max_num_seqs=4, max_num_batched_tokens=32)
    want = [o.outputs[0].token_ids for o in roomy.generate(prompts, sp)]
    tight = LLM(folder, dtype="float32", device="cpu", block_size=8, num_blocks=14, max_model_len=128,
                max_num_seqs=4, max_num_batched_tokens=32)
    outs = tight.generate(prompts, sp)
    assert sum(o.num_preemptions for o in outs) > 0, "the pool was meant to be too small"
    assert [o.outputs[0].token_ids for o in outs] == want
    tight.engine.cache.check()
    assert tight.engine.cache.num_free_pages() == [14, 14]


def test_running_a_step_ahead_gives_the_same_tokens(emulated):
    """Decode steps launched before the previous step's ids are read (tokens taken on the device)
    produce what one-step-at-a-time produces, also when requests stop on a token or at different
    lengths while a step ahead of them is already running."""
    folder = model_folder("tiny_qwen2")
    cfg = load_config(folder)
    prompts = list(random_requests(cfg.vocab_size, (30, 9, 26, 20, 3), seed=6).values())

    def run(ahead, stop, **kw):
        sps = [SamplingParams(temperature=0.8 if i % 2 else 0.0, seed=50 + i, max_tokens=10 + 3 * i,
                              stop_token_ids=stop, ignore_eos=True) for i in range(len(prompts))]
        args = dict(dtype="float32", device="cpu", block_size=8, num_blocks=64, max_model_len=128, max_num_seqs=5,
                    max_num_batched_tokens=64, async_scheduling=ahead)
        args.update(kw)
        llm = LLM(folder, **args)
        steps_ahead = 0
        reqs = [llm.add_request(p, sp) for p, sp in zip(prompts, sps)]
        while llm.scheduler.has_unfinished():
            llm.step()
            steps_ahead += llm._in_flight is not None
        llm.engine.cache.check()
        assert not llm.engine.cache.requests
        return [(r.output, r.finish_reason) for r in reqs], steps_ahead

    free, _ = run(False, [])
    stop = [free[1][0][4], free[3][0][7]]              # tokens that two requests produce midway
    want, none_ahead = run(False, stop)
    assert none_ahead == 0 and {"stop", "length"} == {r for _, r in want}
    got, ahead = run(True, stop)
    assert ahead > 10, "decode steps were meant to be launched ahead"
    assert got == want
    # with fewer request slots than requests, and with so few pages that requests are pre-empted
    assert run(True, stop, max_num_seqs=2)[0] == want
    assert run(True, stop, num_blocks=16)[0] == want


def test_padding_rows_of_a_graph_bucket_change_nothing(emulated):
    """pack(pad_to=...) is what CUDA-graph decode steps run on: padded rows must not write to the
    cache, read a block table or change the real rows' logits."""
    from rvllm_b200.engine import StepEntry
    folder = model_folder("tiny_qwen2")
    cfg = load_config(folder)
    reqs = random_requests(cfg.vocab_size, (20, 9, 13), seed=1)
    eng = trace_mod.build_engine(folder, "float32", 3 * 64, block_size=8, device="cpu")
    r = eng.runner
    for rid, toks in reqs.items():
        r.step([StepEntry(rid, toks, [])])
    entries = [StepEntry(rid, [5], [0]) for rid in reqs]
    r.validate(entries)
    starts = r.reserve(entries)
    before = [g.tensor.clone() for g in eng.cache.groups]
    ctx_plain = r.pack(entries, starts)
    a = eng.model.compute_logits(eng.model.forward(ctx_plain, eng.cache), ctx_plain).clone()
    after_plain = [g.tensor.clone() for g in eng.cache.groups]
    for g, b in zip(eng.cache.groups, before):
        g.tensor.copy_(b)
    ctx_pad = r.pack(entries, starts, pad_to=8)        # reuses the metadata buffer of the step
    assert ctx_pad.num_seqs == 8 and ctx_pad.num_tokens == 8 and ctx_pad.attention[0].block_tables.shape == (8, r.max_blocks)
    assert ctx_pad.attention[0].ctx_lens.tolist()[3:] == [0] * 5
    assert ctx_pad.attention[0].slot_mapping.tolist()[3:] == [-1] * 5 and ctx_pad.state_slots.tolist()[3:] == [-1] * 5
    b_ = eng.model.compute_logits(eng.model.forward(ctx_pad, eng.cache), ctx_pad)
    assert torch.allclose(a, b_[:3], rtol=0, atol=1e-6)     # the CPU product rounds differently for 8 rows
    for g, ap in zip(eng.cache.groups, after_plain):
        assert torch.allclose(g.tensor, ap, rtol=0, atol=1e-6)


def test_step_refuses_bad_input_and_stays_usable(emulated):
    from rvllm_b200 import KvExhausted, SchedulerError
    from rvllm_b200.engine import StepEntry
    eng = trace_mod.build_engine(model_folder("tiny_llama"), "float32", 64, block_size=16, device="cpu")
    r = eng.runner
    with pytest.raises(SchedulerError, match="vocabulary"):
        r.step([StepEntry("a", [1, 9999], [0])])
    with pytest.raises(SchedulerError, match="no tokens"):
        r.step([StepEntry("a", [], [])])
    with pytest.raises(SchedulerError, match="wanted place"):
        r.step([StepEntry("a", [1, 2], [2])])
    with pytest.raises(SchedulerError, match="twice"):
        r.step([StepEntry("a", [1], []), StepEntry("a", [2], [])])
    with pytest.raises(SchedulerError, match="max_model_len"):
        r.step([StepEntry("a", [1] * 65, [])])
    with pytest.raises(KvExhausted):
        r.step([StepEntry("a", [1] * 40, []), StepEntry("b", [1] * 40, [])])
    assert not eng.cache.requests and eng.cache.num_free_pages() == [4]    # nothing was taken by the refused steps
    out = r.step([StepEntry("a", [1, 2, 3], [2])])
    assert out.shape == (1, 261) and torch.isfinite(out).all()
