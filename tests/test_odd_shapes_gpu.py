"""Unusual sizes through the whole engine on the GPU: head sizes that are no power of two, groups
of 1, 5, 8 and 20 query heads per kv head, widths that are no multiple of 8 or 16, odd
vocabularies, windows, biases.  Every kernel either serves the size or hands it to a kernel
that does; the logits are compared with the plain implementation under two ways of cutting
(whole, and mixed with pages used again), in float32 and bfloat16."""
import io
import tempfile

import pytest
import torch

import plain_impl
import trace_tools as TT
from model_tools import random_requests

pytestmark = pytest.mark.gpu


def cfg(arch, H, L, nh, nkv, hd, I, V, **kw):
    c = {"architectures": [arch], "hidden_size": H, "num_hidden_layers": L, "num_attention_heads": nh,
         "num_key_value_heads": nkv, "head_dim": hd, "intermediate_size": I, "vocab_size": V,
         "max_position_embeddings": 512, "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "tie_word_embeddings": False,
         "hidden_act": "silu", "torch_dtype": "bfloat16"}
    c.update(kw)
    return c


ODD = {
    "hd48_group2": cfg("LlamaForCausalLM", 120, 2, 6, 3, 48, 200, 300),
    "hd80_bias_tied": cfg("Qwen2ForCausalLM", 328, 2, 4, 4, 80, 264, 515, tie_word_embeddings=True, rms_norm_eps=1e-6),
    "hd128_group8_window": cfg("Qwen2ForCausalLM", 256, 3, 8, 1, 128, 512, 1000, use_sliding_window=True, sliding_window=48,
                               layer_types=["sliding_attention", "full_attention", "sliding_attention"]),
    "hd16_group20": cfg("LlamaForCausalLM", 96, 2, 20, 1, 16, 172, 261),
    "llama_with_biases": cfg("LlamaForCausalLM", 128, 2, 4, 2, 32, 172, 261, attention_bias=True),   # q, k, v and o
    "width100_group5": cfg("LlamaForCausalLM", 100, 2, 10, 2, 112, 172, 333, rope_theta=500000.0),
    "hd64_many_heads": cfg("LlamaForCausalLM", 192, 2, 12, 4, 64, 344, 640,
                           rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                         "high_freq_factor": 4.0, "original_max_position_embeddings": 64}),
}

_folders = {}


def folder_of(name):
    import rvllm_b200
    if name not in _folders:
        d = tempfile.TemporaryDirectory(prefix=f"rvllm_odd_{name}_")
        rvllm_b200.write_random_model(rvllm_b200.config_from_dict(ODD[name]), d.name, seed=3, dtype="bfloat16")
        _folders[name] = d
    return _folders[name].name


@pytest.mark.parametrize("dtype,tol", [("float32", 1e-4), ("bfloat16", 2e-2)])
@pytest.mark.parametrize("name", sorted(ODD))
def test_odd_shapes_match_plain(name, dtype, tol, tmp_path):
    from rvllm_b200.engine import trace as trace_mod
    folder = folder_of(name)
    conf, w = plain_impl.read_model_folder(folder)
    vocab = conf["vocab_size"]
    reqs = random_requests(vocab, (3, 70, 129, 40, 17), seed=5)
    ref = {rid: plain_impl.forward(conf, w, toks) for rid, toks in reqs.items()}
    for schedule, build in (("bulk_tail", lambda: TT.schedule_bulk_tail(reqs, tail=20)),
                            ("mixed", lambda: TT.schedule_mixed(reqs, live=3, seed=1))):
        trace = build()
        engine = trace_mod.build_engine(folder, dtype, trace.max_tokens, block_size=16, max_live=4)
        out = tmp_path / f"{schedule}"
        n = trace_mod.replay(engine, io.StringIO(trace.lines()), str(out))
        assert n == len(trace.steps)
        got = TT.read_logits(str(out), trace, vocab)
        TT.compare(got, ref, tol, f"{name}/{dtype}/{schedule}")
        engine.cache.check()
        assert not engine.cache.requests


@pytest.mark.parametrize("name", ["hd48_group2", "hd16_group20", "width100_group5"])
def test_odd_shapes_generate_with_graphs(name):
    """Decode steps from CUDA graphs (padded buckets, the decode kernels) against eager steps."""
    from rvllm_b200 import LLM, SamplingParams
    folder = folder_of(name)
    vocab = ODD[name]["vocab_size"]
    prompts = list(random_requests(vocab, (5, 33, 18), seed=2).values())
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    outs = {}
    for eager in (True, False):
        llm = LLM(folder, dtype="float32", block_size=16, num_blocks=64, max_model_len=128, max_num_seqs=4,
                  max_num_batched_tokens=64, enforce_eager=eager)
        outs[eager] = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert outs[True] == outs[False]
    conf, w = plain_impl.read_model_folder(folder)
    for p, toks in zip(prompts, outs[True]):
        assert toks == plain_impl.greedy_generate(conf, w, p, 12)
