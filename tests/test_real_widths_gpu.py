"""The whole engine at the layer widths it is measured at: two layers of Llama-3.1-8B's sizes
(hidden 4,096, 32 query and 8 key/value heads of 128, feed-forward 14,336, llama3 rotary scaling)
and two of Qwen2.5-7B's (hidden 3,584, 28 / 4 heads, q/k/v bias, feed-forward 18,944), only the
vocabulary cut to 8,192 - through bin/trace_run against the plain implementation, in float32 and
bfloat16: requests whole and mixed (with the large prefill tiles and a pre-emption in it), decode
steps replayed from CUDA graphs, 40 and 64 sequences decoded at once, and contexts that cross
the context buckets of the decode graphs.

The plain implementation's float64 arithmetic runs on the GPU here (torch as an array library):
on the CPU these widths would take minutes.

float32 must agree to 1e-4 of each position's largest logit.  For bfloat16 a constant would be a
guess: at these widths the rounding of stored activations alone moves a position's logits by 1.2 %
of its largest logit in the median and 1.8 % at worst (the plain implementation shows it when it
rounds what an engine would store).  So the yardstick is measured on the same requests, and the
engine may exceed its worst position by half and its median by a quarter
(trace_tools.compare_bfloat16)."""
import pytest

import trace_tools as TT
from model_tools import folder_for, plain_logits, random_requests

pytestmark = pytest.mark.gpu

TOL = {"float32": 1e-4}
VOCAB = 8192

WIDTHS = {
    "llama31_8b": {
        "architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "num_hidden_layers": 2, "num_attention_heads": 32,
        "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "vocab_size": VOCAB,
        "max_position_embeddings": 4096, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 8192},
        "attention_bias": False, "tie_word_embeddings": False, "hidden_act": "silu", "torch_dtype": "bfloat16"},
    "qwen25_7b": {
        "architectures": ["Qwen2ForCausalLM"], "hidden_size": 3584, "num_hidden_layers": 2, "num_attention_heads": 28,
        "num_key_value_heads": 4, "head_dim": 128, "intermediate_size": 18944, "vocab_size": VOCAB,
        "max_position_embeddings": 4096, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "use_sliding_window": False,
        "tie_word_embeddings": False, "hidden_act": "silu", "torch_dtype": "bfloat16"},
}

_cache = {}


def model_and_reference(name, lengths, seed):
    """(folder, requests, plain float64 logits, the same with bfloat16 storage) - the folder is
    written once per test session, the logits once per (model, requests)."""
    if name not in _cache:
        _cache[name] = folder_for(WIDTHS[name], seed=11)
    folder = _cache[name]
    key = (name, tuple(lengths), seed)
    if key not in _cache:
        reqs = random_requests(VOCAB, lengths, seed=seed)
        _cache[key] = (reqs,) + plain_logits(folder, reqs, device="cuda", rounded=True)
    return (folder,) + _cache[key]


def check(got, ref, rounded, dtype, what):
    if dtype == "float32":
        TT.compare(got, ref, TOL[dtype], what)
    else:
        TT.compare_bfloat16(got, ref, rounded, what)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(WIDTHS))
def test_whole_and_mixed_at_real_widths(tmp_path, name, dtype):
    """Prompts of 300 / 700 / 520 tokens take the prefill GEMM on single CTAs and on pairs, the
    mixed schedule brings portions of 130 to 300 tokens beside decoded tokens of other requests."""
    folder, reqs, ref, rounded = model_and_reference(name, (300, 45, 700, 129, 520, 77), seed=21)
    for schedule, trace in (("whole", TT.schedule_whole(reqs)),
                            ("mixed", TT.schedule_mixed(reqs, seed=2, portions=(2, 40, 130, 260, 300)))):
        out = tmp_path / schedule
        TT.run_trace_tool(folder, dtype, trace, str(out))
        got = TT.read_logits(str(out), trace, VOCAB)
        check(got, ref, rounded, dtype, f"{name}/{schedule}/{dtype}")


def many_decoding_at_once(reqs, prompt_of, counts=(64, 40), steps=6):
    """Prompts whole, sixteen requests a step; then `steps` decode steps with all of them, then
    some are ended and the rest decode on (64, then 40 sequences at once)."""
    t = TT.Trace()
    ids = list(reqs)
    for i in range(0, len(ids), 16):
        t.add([(rid, reqs[rid][:prompt_of[rid]], 0) for rid in ids[i:i + 16]])
    pos = dict(prompt_of)
    live = list(ids)
    for n_live in counts:
        ended, live = live[n_live:], live[:n_live]
        if ended:
            # a step of their own ends the dropped requests: one more token each
            t.add([(rid, reqs[rid][pos[rid]:pos[rid] + 1], pos[rid]) for rid in ended], end=ended)
        for _ in range(steps):
            t.add([(rid, reqs[rid][pos[rid]:pos[rid] + 1], pos[rid]) for rid in live])
            for rid in live:
                pos[rid] += 1
    t.add([(rid, reqs[rid][pos[rid]:pos[rid] + 1], pos[rid]) for rid in live], end=live)
    return t


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(WIDTHS))
def test_forty_and_sixty_four_sequences_decode_from_graphs(tmp_path, name, dtype):
    """Decode batches of 64 and 40 rows (in bfloat16 the products of 33 to 64 rows and the rotary
    kernel after them), replayed from CUDA graphs after each bucket's first step."""
    lengths = [20 + (7 * i) % 41 for i in range(64)]
    folder, reqs, ref, rounded = model_and_reference(name, [n + 14 for n in lengths], seed=22)
    prompt_of = {rid: n for rid, n in zip(reqs, lengths)}
    trace = many_decoding_at_once(reqs, prompt_of)
    fed = {rid: sum(1 for rows in trace.rows.values() for r, _ in rows if r == rid) for rid in ref}
    ref, rounded = ({rid: t[rid][:fed[rid]] for rid in t} for t in (ref, rounded))
    TT.run_trace_tool(folder, dtype, trace, str(tmp_path), extra=("--graphs", "--max-live", "64"))
    got = TT.read_logits(str(tmp_path), trace, VOCAB)
    check(got, ref, rounded, dtype, f"{name}/decode 64 and 40/{dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_contexts_cross_the_graph_buckets(tmp_path, dtype):
    """A decode graph is laid out for contexts up to 512, 768, 1,024, 1,536, 2,048 tokens (the
    attention's split of the keys is frozen in it).  Four requests decode across one boundary each,
    alone, and then two of them together across two more."""
    name = "llama31_8b"
    prompts = {"r0": 500, "r1": 760, "r2": 1015, "r3": 1530, "r4": 505, "r5": 1020}
    folder, reqs, ref, rounded = model_and_reference(name, [n + 24 for n in prompts.values()], seed=23)
    t = TT.Trace()
    for rid in ("r0", "r1", "r2", "r3"):
        n, toks = prompts[rid], reqs[rid]
        t.add([(rid, toks[:n], 0)])
        for i in range(n, len(toks)):
            t.add([(rid, toks[i:i + 1], i)], end=[rid] if i == len(toks) - 1 else [])
    t.add([("r4", reqs["r4"][:505], 0), ("r5", reqs["r5"][:1020], 0)])
    for i in range(24):
        last = i == 23
        t.add([("r4", reqs["r4"][505 + i:506 + i], 505 + i), ("r5", reqs["r5"][1020 + i:1021 + i], 1020 + i)],
              end=["r4", "r5"] if last else [])
    TT.run_trace_tool(folder, dtype, t, str(tmp_path), extra=("--graphs",))
    got = TT.read_logits(str(tmp_path), t, VOCAB)
    check(got, ref, rounded, dtype, f"{name}/graph context buckets/{dtype}")


# One layer at the widths of other checkpoints of the two architectures (vocabulary cut): head size 64, groups of
# 4, 5, 6, 7 and 8 query heads a key/value head, hidden sizes whose products have 7, 12, 16, 40 and 64 tiles of 128
# features, tied embeddings.  Each meets another side of the kernels' dispatch: how K is split, which tile the
# attention packs, which epilogue rotates.
OTHER_WIDTHS = {
    "llama32_1b": dict(arch="LlamaForCausalLM", hidden=2048, heads=32, kv=8, hd=64, inter=8192, tie=True, theta=500000.0, eps=1e-5),
    "qwen25_05b": dict(arch="Qwen2ForCausalLM", hidden=896, heads=14, kv=2, hd=64, inter=4864, tie=True, theta=1000000.0, eps=1e-6),
    "qwen25_15b": dict(arch="Qwen2ForCausalLM", hidden=1536, heads=12, kv=2, hd=128, inter=8960, tie=True, theta=1000000.0, eps=1e-6),
    "qwen25_14b": dict(arch="Qwen2ForCausalLM", hidden=5120, heads=40, kv=8, hd=128, inter=13824, tie=False, theta=1000000.0, eps=1e-6),
    "llama31_70b": dict(arch="LlamaForCausalLM", hidden=8192, heads=64, kv=8, hd=128, inter=28672, tie=False, theta=500000.0, eps=1e-5),
}
OTHER_VOCAB = 4099


def other_config(w):
    cfg = {"architectures": [w["arch"]], "hidden_size": w["hidden"], "num_hidden_layers": 1, "num_attention_heads": w["heads"],
           "num_key_value_heads": w["kv"], "head_dim": w["hd"], "intermediate_size": w["inter"], "vocab_size": OTHER_VOCAB,
           "max_position_embeddings": 2048, "rms_norm_eps": w["eps"], "rope_theta": w["theta"], "tie_word_embeddings": w["tie"],
           "hidden_act": "silu", "torch_dtype": "bfloat16"}
    if w["arch"] == "Qwen2ForCausalLM":
        cfg["use_sliding_window"] = False
    else:
        cfg["attention_bias"] = False
    return cfg


@pytest.mark.parametrize("name", sorted(OTHER_WIDTHS))
def test_one_layer_at_the_widths_of_other_checkpoints(tmp_path, name):
    """bfloat16, prompts of 150 / 33 / 260 / 70 / 400 tokens whole (the short-prompt products in blocks of 128 rows,
    the narrow prefill tiles) and in mixed portions beside decoded tokens, against the plain implementation."""
    folder = folder_for(other_config(OTHER_WIDTHS[name]), seed=12)
    reqs = random_requests(OTHER_VOCAB, (150, 33, 260, 70, 400), seed=31)
    ref, rounded = plain_logits(folder, reqs, device="cuda", rounded=True)
    for schedule, trace in (("whole", TT.schedule_whole(reqs)),
                            ("mixed", TT.schedule_mixed(reqs, seed=5, portions=(2, 40, 130, 200)))):
        out = tmp_path / schedule
        TT.run_trace_tool(folder, "bfloat16", trace, str(out))
        got = TT.read_logits(str(out), trace, OTHER_VOCAB)
        TT.compare_bfloat16(got, ref, rounded, f"{name}/{schedule}")
