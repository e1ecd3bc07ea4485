"""Continuous batching under load: many requests of uneven length, small token budgets, few pages.
In float32 the kernels sum every row in an order that does not depend on the batch, so the generated
tokens must be identical however the scheduler cuts and mixes the work."""
import pytest
import torch

import tiny_configs

pytestmark = pytest.mark.gpu

MID = {
    "architectures": ["Qwen2ForCausalLM"], "hidden_size": 256, "num_hidden_layers": 3, "num_attention_heads": 8,
    "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 688, "vocab_size": 1000,
    "max_position_embeddings": 2048, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "tie_word_embeddings": False,
    "hidden_act": "silu", "torch_dtype": "bfloat16", "use_sliding_window": True, "sliding_window": 300,
    "layer_types": ["full_attention", "sliding_attention", "full_attention"],
}


def run(dtype, prompts, sp, **kw):
    from rvllm_b200 import LLM, config_from_dict
    args = dict(config=config_from_dict(dict(MID)), random_weights=True, seed=1, dtype=dtype, block_size=16,
                max_model_len=1024, max_num_seqs=16, max_num_batched_tokens=512)
    args.update(kw)
    llm = LLM(**args)
    outs = llm.generate(prompts, sp)
    llm.engine.cache.check()
    assert not llm.engine.cache.requests
    return [o.outputs[0].token_ids for o in outs], sum(o.num_preemptions for o in outs), llm


def test_float32_tokens_do_not_depend_on_scheduling():
    from rvllm_b200 import SamplingParams
    g = torch.Generator().manual_seed(0)
    lengths = torch.randint(8, 700, (24,), generator=g).tolist()
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in lengths]
    sp = [SamplingParams(temperature=0.0 if i % 2 else 0.9, top_p=0.95, seed=100 + i, max_tokens=24 + (i % 5) * 8,
                         ignore_eos=True) for i in range(len(prompts))]
    base, _, _ = run("float32", prompts, sp, num_blocks=2048, max_num_seqs=24, max_num_batched_tokens=4096)
    cut, _, _ = run("float32", prompts, sp, num_blocks=2048, max_num_seqs=5, max_num_batched_tokens=96, max_prefill_chunk=64)
    assert cut == base
    tight, preempted, _ = run("float32", prompts, sp, num_blocks=120, max_num_seqs=8, max_num_batched_tokens=300)
    assert preempted > 0, "the pool was meant to force pre-emption"
    assert tight == base


def test_bfloat16_mixed_batches_run_clean_and_repeat():
    """The serving kernels under the same load (tcgen05 attention and GEMMs for prompt portions beside
    decode kernels, CUDA graphs and eager steps alternating): no error, no lost page, and the same
    tokens when the same schedule is run twice."""
    from rvllm_b200 import SamplingParams
    g = torch.Generator().manual_seed(1)
    lengths = torch.randint(8, 900, (32,), generator=g).tolist()
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in lengths]
    sp = SamplingParams(temperature=0.7, seed=7, max_tokens=40, ignore_eos=True)
    a, _, llm = run("bfloat16", prompts, sp, num_blocks=600, max_num_seqs=16, max_num_batched_tokens=384)
    assert llm.engine.runner._graphs, "decode steps should have been replayed from graphs"
    b, _, _ = run("bfloat16", prompts, sp, num_blocks=600, max_num_seqs=16, max_num_batched_tokens=384)
    assert a == b
    assert all(len(t) == 40 for t in a)


def test_bfloat16_batch_of_32_in_one_chain_of_dependent_launches():
    """32 sequences of 8 kv heads decode together: the evenly cut attention kernel and its merge
    kernel run between this project's own GEMMs (cluster reduce, rotation in the epilogue), every
    kernel launched while its predecessor still runs.  A kernel that wrote before its wait for the
    predecessor once corrupted a buffer still in use; so: no error, the same tokens twice, and the
    same tokens as with eager steps - except that a graph, laid out for its bucket's longest context,
    may split the keys differently from an eager step, so a request may part from its eager run at a
    token whose two best logits lie within bfloat16's reach of one another (checked), nowhere else."""
    from rvllm_b200 import SamplingParams
    wide = dict(MID, num_attention_heads=16, num_key_value_heads=8, head_dim=32, hidden_size=512)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 1000, (int(n),), generator=g).tolist() for n in torch.randint(100, 400, (32,), generator=g)]
    sp = SamplingParams(temperature=0.0, max_tokens=48, ignore_eos=True)

    def go(**extra):
        from rvllm_b200 import LLM, config_from_dict
        llm = LLM(config=config_from_dict(dict(wide)), random_weights=True, seed=3, dtype="bfloat16", block_size=16,
                  max_model_len=1024, num_blocks=1600, max_num_seqs=32, max_num_batched_tokens=2048, **extra)
        outs = llm.generate(prompts, sp)
        llm.engine.cache.check()
        return [o.outputs[0].token_ids for o in outs], llm

    a, llm = go()
    assert any(k[0] == 32 for k in llm.engine.runner._graphs), "the 32-row decode graph should have been used"
    b, _ = go()
    assert a == b
    c, eager = go(enforce_eager=True)
    from rvllm_b200.engine import StepEntry
    parted = 0
    for prompt, ta, tc in zip(prompts, a, c):
        j = next((i for i in range(len(ta)) if ta[i] != tc[i]), None)
        if j is None:
            continue
        parted += 1
        ids = list(prompt) + ta[:j]
        logits = eager.engine.runner.step([StepEntry("margin", ids, [len(ids) - 1])])[0].float()
        eager.engine.runner.finish("margin")
        top = torch.topk(logits, 2)
        assert {ta[j], tc[j]} == set(top.indices.tolist()), "the two runs chose the two best tokens"
        assert float(top.values[0] - top.values[1]) / float(logits.abs().max()) < 2e-2, "and these lie within rounding"
    assert parted <= 3
