"""Generation through the Python entry point on the GPU."""
import pytest
import torch

import plain_impl
from model_tools import model_folder, random_requests

pytestmark = pytest.mark.gpu


def make_llm(name, dtype, **kw):
    from rvllm_b200 import LLM
    args = dict(dtype=dtype, block_size=8, num_blocks=96, max_model_len=256, max_num_seqs=4, max_num_batched_tokens=48)
    args.update(kw)
    return LLM(model_folder(name), **args)


@pytest.mark.parametrize("name", ["tiny_llama", "tiny_qwen2"])
def test_greedy_float32_equals_plain(name):
    from rvllm_b200 import SamplingParams
    cfg, w = plain_impl.read_model_folder(model_folder(name))
    prompts = list(random_requests(cfg["vocab_size"], (5, 17, 33, 60, 2), seed=2).values())
    llm = make_llm(name, "float32", max_prefill_chunk=16)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.outputs[0].token_ids == plain_impl.greedy_generate(cfg, w, p, 10)
    llm.engine.cache.check()
    assert not llm.engine.cache.requests


@pytest.mark.parametrize("name", ["tiny_llama", "tiny_qwen2"])
def test_greedy_bfloat16_follows_plain_where_the_margin_allows(name):
    """bfloat16 may flip a token only where the plain logits' two best are closer than its error."""
    from rvllm_b200 import SamplingParams
    cfg, w = plain_impl.read_model_folder(model_folder(name))
    prompts = list(random_requests(cfg["vocab_size"], (9, 40, 70), seed=5).values())
    llm = make_llm(name, "bfloat16")
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    for p, o in zip(prompts, outs):
        ids = list(p)
        for tok in o.outputs[0].token_ids:
            logits = plain_impl.forward(cfg, w, ids)[-1]
            top = torch.topk(logits, 2).values
            margin = float(top[0] - top[1]) / float(logits.abs().max())
            if margin > 4e-2:
                assert tok == int(logits.argmax()), f"flipped at a margin of {margin:.3f}"
            ids.append(tok)                                  # follow the engine's own continuation


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuda_graph_decode_equals_eager_and_batching_does_not_change_samples(dtype):
    """float32: the same tokens from eager steps, from graph replays (padded batches) and from one
    request at a time under a tiny token budget.  bfloat16: a graph is laid out for its bucket's
    longest context, so its attention may split the keys differently from an eager step and its sums
    may differ in the last bit; two runs may then part ways, but only at a draw whose uniform lies
    within bfloat16's reach of a step of the CDF (checked with the plain sampler on the plain logits
    of the common prefix)."""
    from rvllm_b200 import SamplingParams
    cfg, w = plain_impl.read_model_folder(model_folder("tiny_qwen2"))
    prompts = list(random_requests(cfg["vocab_size"], (5, 23, 70, 9, 41), seed=8).values())
    sp = SamplingParams(temperature=0.8, top_k=40, seed=3, max_tokens=24, ignore_eos=True)
    eager = make_llm("tiny_qwen2", dtype, enforce_eager=True, max_num_seqs=8)
    a = [o.outputs[0].token_ids for o in eager.generate(prompts, sp)]
    graphs = make_llm("tiny_qwen2", dtype, enforce_eager=False, max_num_seqs=8)
    b = [o.outputs[0].token_ids for o in graphs.generate(prompts, sp)]
    assert graphs.engine.runner._graphs, "no decode step was replayed from a graph"
    if dtype == "float32":
        assert a == b
        # other portions, other batches: one request at a time, tiny token budget
        alone = make_llm("tiny_qwen2", dtype, max_num_seqs=1, max_num_batched_tokens=7)
        c = [o.outputs[0].token_ids for o in alone.generate(prompts, sp)]
        assert a == c
        return
    same = 0
    for p, ta, tb in zip(prompts, a, b):
        j = next((i for i in range(len(ta)) if ta[i] != tb[i]), None)
        if j is None:
            same += 1
            continue
        logits = plain_impl.forward(cfg, w, list(p) + ta[:j])[-1]
        _, margin = plain_impl.sample(logits, 0.8, 3, j, top_k=40)
        assert margin < 2e-2, f"the runs part at output {j} although the draw is {margin:.3f} away from any step of the CDF"
    assert same >= 3, "most requests do not meet such a draw within 24 tokens"


@pytest.mark.parametrize("eager", [False, True])
def test_running_a_step_ahead_gives_the_same_tokens(eager):
    """Decode steps launched before the previous step's ids reach the host take their tokens on the
    device (late_tokens kernel, then the graph or the eager step): same tokens and finish reasons as
    one step at a time, with requests that stop on a token or at different lengths meanwhile."""
    from rvllm_b200 import SamplingParams
    cfg, _ = plain_impl.read_model_folder(model_folder("tiny_qwen2"))
    prompts = list(random_requests(cfg["vocab_size"], (30, 9, 26, 20, 3, 50), seed=6).values())

    def run(ahead, stop, dtype="float32", same_length=False, **kw):
        sps = [SamplingParams(temperature=0.8 if i % 2 else 0.0, seed=50 + i, max_tokens=20 if same_length else 10 + 4 * i,
                              stop_token_ids=stop, ignore_eos=True) for i in range(len(prompts))]
        llm = make_llm("tiny_qwen2", dtype, max_num_seqs=8, max_num_batched_tokens=128, async_scheduling=ahead,
                       enforce_eager=eager, **kw)
        reqs = [llm.add_request(p, sp) for p, sp in zip(prompts, sps)]
        ahead_steps = 0
        while llm.scheduler.has_unfinished():
            llm.step()
            ahead_steps += llm._in_flight is not None
        llm.engine.cache.check()
        assert not llm.engine.cache.requests
        return [(r.output, r.finish_reason) for r in reqs], ahead_steps

    free, _ = run(False, ())
    stop = (free[1][0][4], free[3][0][7])
    want, n0 = run(False, stop)
    got, n1 = run(True, stop)
    assert n0 == 0 and n1 > 10
    assert got == want and {"stop", "length"} == {r for _, r in want}
    assert run(True, stop, num_blocks=24)[0] == want          # few pages: pre-emption in between
    # bfloat16, where the make-up of every batch is the same in both modes
    assert run(True, (), "bfloat16", True)[0] == run(False, (), "bfloat16", True)[0]


def test_finish_reasons_and_stop_tokens():
    from rvllm_b200 import SamplingParams
    cfg, w = plain_impl.read_model_folder(model_folder("tiny_llama"))
    prompt = random_requests(cfg["vocab_size"], (12,), seed=6)["r0"]
    free_run = plain_impl.greedy_generate(cfg, w, prompt, 8)
    llm = make_llm("tiny_llama", "float32")
    out = llm.generate([prompt], SamplingParams(max_tokens=8, stop_token_ids=(free_run[3],), ignore_eos=True))[0]
    first = free_run.index(free_run[3])
    assert out.outputs[0].token_ids == free_run[:first + 1] and out.outputs[0].finish_reason == "stop"
    out = llm.generate([prompt], SamplingParams(max_tokens=5, ignore_eos=True))[0]
    assert out.outputs[0].finish_reason == "length" and len(out.outputs[0].token_ids) == 5


def test_preemption_on_the_gpu_keeps_outputs():
    from rvllm_b200 import SamplingParams
    cfg, _ = plain_impl.read_model_folder(model_folder("tiny_qwen2"))
    prompts = list(random_requests(cfg["vocab_size"], (30, 28, 26, 20), seed=4).values())
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    roomy = make_llm("tiny_qwen2", "float32", num_blocks=64, max_num_batched_tokens=32)
    want = [o.outputs[0].token_ids for o in roomy.generate(prompts, sp)]
    tight = make_llm("tiny_qwen2", "float32", num_blocks=14, max_num_batched_tokens=32)
    outs = tight.generate(prompts, sp)
    assert sum(o.num_preemptions for o in outs) > 0
    assert [o.outputs[0].token_ids for o in outs] == want
    tight.engine.cache.check()


def test_random_weights_without_a_folder_and_loud_errors():
    import tiny_configs
    from rvllm_b200 import ConfigError, KvExhausted, LLM, SamplingParams, config_from_dict
    cfg = config_from_dict(tiny_configs.get("baseline1"))
    llm = LLM(config=cfg, random_weights=True, seed=4, dtype="bfloat16", num_blocks=4, max_model_len=128, max_num_seqs=2)
    out = llm.generate([[1, 2, 3]], SamplingParams(max_tokens=4, ignore_eos=True))[0]
    assert len(out.outputs[0].token_ids) == 4
    with pytest.raises(KvExhausted):
        llm.generate([[1] * 100], SamplingParams(max_tokens=400))       # 128 tokens would need 8 pages; there are 4
    with pytest.raises(ConfigError):
        LLM(config=cfg)                                                  # no folder and no random weights
    with pytest.raises(ConfigError, match="tokenizer"):
        llm.generate(["text needs a tokenizer"], SamplingParams())


def test_graphs_captured_ahead_change_nothing():
    """Decode graphs captured before any request (all batch buckets, contexts up to a limit) are the
    ones the steps then replay: same tokens as with graphs captured on the way, no capture later."""
    from rvllm_b200 import SamplingParams
    cfg, _ = plain_impl.read_model_folder(model_folder("tiny_qwen2"))
    prompts = list(random_requests(cfg["vocab_size"], (5, 23, 70, 9), seed=8).values())
    sp = SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True)
    lazy = make_llm("tiny_qwen2", "bfloat16", max_num_seqs=8)
    want = [o.outputs[0].token_ids for o in lazy.generate(prompts, sp)]
    early = make_llm("tiny_qwen2", "bfloat16", max_num_seqs=8)
    n = early.capture_graphs()
    assert n == len(early.engine.runner._graphs) and n >= 4
    assert early.capture_graphs() == 0                                     # nothing left to capture
    got = [o.outputs[0].token_ids for o in early.generate(prompts, sp)]
    assert got == want and len(early.engine.runner._graphs) == n
    early.engine.cache.check()


def test_benchmark_configuration_0_workload():
    """Tiny Llama-style configuration (2 layers, hidden 64, 4 query / 2 kv heads of 16, block 16):
    prompts of 5, 17 and 33 tokens, 8 greedy tokens each; float32 tokens equal the plain ones,
    bfloat16 tokens follow them where the margin allows."""
    from rvllm_b200 import LLM, SamplingParams
    folder = model_folder("baseline0")
    cfg, w = plain_impl.read_model_folder(folder)
    prompts = list(random_requests(cfg["vocab_size"], (5, 17, 33), seed=0).values())
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    for dtype in ("float32", "bfloat16"):
        llm = LLM(folder, dtype=dtype, block_size=16, num_blocks=12, max_model_len=128, max_num_seqs=3)
        outs = llm.generate(prompts, sp)
        for p, o in zip(prompts, outs):
            got = o.outputs[0].token_ids
            assert len(got) == 8
            if dtype == "float32":
                assert got == plain_impl.greedy_generate(cfg, w, p, 8)
                continue
            ids = list(p)
            for tok in got:
                logits = plain_impl.forward(cfg, w, ids)[-1]
                top = torch.topk(logits, 2).values
                if float(top[0] - top[1]) / float(logits.abs().max()) > 4e-2:
                    assert tok == int(logits.argmax())
                ids.append(tok)
        llm.engine.cache.check()
        assert not llm.engine.cache.requests


def test_benchmark_configuration_1_workload():
    """Tiny Qwen2-style configuration (3 layers, 3 query heads on 1 kv head of 32, bias, tied head,
    block 8): prompts of 1, 9, 40 and 70 tokens fed in portions of 16 beside decoding requests, 12
    tokens each at temperature 0.8 with a seed.  Every sampled token is the plain sampler's for the
    plain logits of the same prefix, unless the uniform lies within rounding of a step of the CDF."""
    from rvllm_b200 import LLM, SamplingParams
    folder = model_folder("baseline1")
    cfg, w = plain_impl.read_model_folder(folder)
    prompts = list(random_requests(cfg["vocab_size"], (1, 9, 40, 70), seed=1).values())
    sps = [SamplingParams(temperature=0.8, seed=1000 + i, max_tokens=12, ignore_eos=True) for i in range(4)]
    llm = LLM(folder, dtype="float32", block_size=8, num_blocks=44, max_model_len=256, max_num_seqs=4,
              max_num_batched_tokens=24, max_prefill_chunk=16)
    outs = llm.generate(prompts, sps)
    checked = 0
    for i, (p, o) in enumerate(zip(prompts, outs)):
        ids = list(p)
        assert len(o.outputs[0].token_ids) == 12
        for j, tok in enumerate(o.outputs[0].token_ids):
            want, margin = plain_impl.sample(plain_impl.forward(cfg, w, ids)[-1], 0.8, 1000 + i, j)
            if margin > 1e-4:
                assert tok == want, f"request {i}, output {j}: {tok} vs the plain sampler's {want} (margin {margin:.1e})"
                checked += 1
            ids.append(tok)
    assert checked >= 40
    llm.engine.cache.check()
    assert not llm.engine.cache.requests
    # the same requests in bfloat16, chunked the same way: runs clean and repeats itself
    a, b = (LLM(folder, dtype="bfloat16", block_size=8, num_blocks=44, max_model_len=256, max_num_seqs=4,
                max_num_batched_tokens=24, max_prefill_chunk=16).generate(prompts, sps) for _ in range(2))
    assert [o.outputs[0].token_ids for o in a] == [o.outputs[0].token_ids for o in b]


def test_a_kernel_that_gave_up_a_wait_fails_the_step_loudly():
    """The tcgen05 kernels bound their waits and report through one status word that the entry point
    reads beside each step's sampled ids (no extra synchronisation).  Nothing on a healthy GPU makes
    a wait run out, so the word is set by hand here: the step must raise instead of returning ids,
    and the word and the split-K arrival counters must be clean afterwards."""
    from rvllm_b200 import KernelError, SamplingParams
    llm = make_llm("tiny_qwen2", "bfloat16")
    K = llm.engine.kernels
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    want = llm.generate([[1, 2, 3, 4, 5]], sp)[0].outputs[0].token_ids
    x = torch.randn(4, 512, device="cuda").bfloat16()
    K.linear_decode(x, torch.randn(256, 512, device="cuda").bfloat16(), splits=2, cluster=False)   # makes the counters
    K._decode_counters[1] = 1                      # as an aborted CTA would leave them
    K.status_word.fill_(3)
    llm.add_request([1, 2, 3, 4, 5], sp)
    with pytest.raises(KernelError, match="bounded wait"):
        while llm.scheduler.has_unfinished():
            llm.step()
    assert int(K.status_word.item()) == 0 and int(K._decode_counters.abs().sum()) == 0
    K.raise_on_abort()                             # clean: nothing to report
    fresh = make_llm("tiny_qwen2", "bfloat16")
    assert fresh.generate([[1, 2, 3, 4, 5]], sp)[0].outputs[0].token_ids == want
