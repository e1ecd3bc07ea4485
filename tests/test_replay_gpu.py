"""Trace replay on the GPU through bin/trace_run, as a user runs it: the same requests whole,
with the last 32 tokens one by one, in portions of changing size, and mixed with other requests
in a pool so small that pages are used again - in float32 and in bfloat16 - against the plain
implementation."""
import os
import subprocess
import sys

import pytest
import torch

import trace_tools as TT
from model_tools import model_folder, plain_logits, random_requests

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")
TOL = {"float32": 1e-4, "bfloat16": 2e-2}
LENGTHS = {"tiny_llama": (45, 70, 133, 81, 200, 38), "tiny_qwen2": (90, 37, 210, 64, 151, 75),
           # the two tiny configurations of the benchmark description: their prompts plus their new tokens
           "baseline0": (5 + 8, 17 + 8, 33 + 8, 100, 128, 64), "baseline1": (1 + 12, 9 + 12, 40 + 12, 70 + 12, 256, 130)}
BLOCK = {"tiny_llama": 16, "tiny_qwen2": 8, "baseline0": 16, "baseline1": 8}
SCHEDULES = {"whole": TT.schedule_whole, "bulk_tail": TT.schedule_bulk_tail, "portions": TT.schedule_portions,
             "mixed": TT.schedule_mixed}
_ref_cache = {}


def reference(name):
    if name not in _ref_cache:
        from rvllm_b200 import load_config
        folder = model_folder(name)
        vocab = load_config(folder).vocab_size
        reqs = random_requests(vocab, LENGTHS[name], seed=3)
        _ref_cache[name] = (folder, vocab, reqs) + plain_logits(folder, reqs, rounded=True)
    return _ref_cache[name][:4]


def check(got, name, dtype, what):
    """float32: 1e-4 of each position's largest logit.  bfloat16: within 2e-2, and measured against
    what storing activations in bfloat16 costs by itself on the same requests (see
    trace_tools.compare_bfloat16)."""
    ref, rounded = _ref_cache[name][3:5]
    TT.compare(got, ref, TOL[dtype], what)
    if dtype == "bfloat16":
        TT.compare_bfloat16(got, ref, rounded, what)


def run_trace(folder, dtype, trace, out_dir, block_size=16, extra=(), in_process=False):
    """Replay with bin/trace_run in a process of its own, or (to save the start-up of a process in a
    large matrix) in this process through the very functions that program calls."""
    if not in_process:
        TT.run_trace_tool(folder, dtype, trace, out_dir, block_size, extra)
        return
    import io
    from rvllm_b200.engine import trace as trace_mod
    engine = trace_mod.build_engine(folder, dtype, trace.max_tokens, block_size, graphs="--graphs" in extra)
    echo = io.StringIO()
    trace_mod.replay(engine, io.StringIO(trace.lines()), out_dir, echo)
    assert echo.getvalue().splitlines() == [f"done {i}" for i in range(len(trace.steps))]
    engine.cache.check()
    assert not engine.cache.requests


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(LENGTHS))
@pytest.mark.parametrize("schedule", list(SCHEDULES))
def test_replay_matches_plain(tmp_path, name, schedule, dtype):
    folder, vocab, reqs, ref = reference(name)
    trace = SCHEDULES[schedule](reqs)
    if schedule == "mixed":
        assert trace.preemptions == 1, "one live request is ended and fed again from position 0"
    run_trace(folder, dtype, trace, str(tmp_path), block_size=BLOCK[name],
              in_process=name.startswith("baseline") and schedule != "mixed")
    got = TT.read_logits(str(tmp_path), trace, vocab)
    check(got, name, dtype, f"{name}/{schedule}/{dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_qwen2", "baseline0"])
def test_mixed_replay_with_decode_graphs(tmp_path, name, dtype):
    """The mixed schedule again with decode-only steps replayed from CUDA graphs (the steps that
    bring portions run eagerly in between): same logits."""
    folder, vocab, reqs, ref = reference(name)
    trace = TT.schedule_mixed(reqs, seed=5)
    run_trace(folder, dtype, trace, str(tmp_path), block_size=BLOCK[name], extra=("--graphs",))
    got = TT.read_logits(str(tmp_path), trace, vocab)
    check(got, name, dtype, f"{name}/mixed with graphs/{dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(tmp_path, dtype):
    """A prompt of two tokens, then 400 tokens one by one: the first positions of a sequence and
    decoding across dozens of pages (and, in the windowed layers, far past the window)."""
    from rvllm_b200 import load_config
    folder = model_folder("tiny_qwen2")
    vocab = load_config(folder).vocab_size
    reqs = random_requests(vocab, (402,), seed=12)
    ref = plain_logits(folder, reqs)
    toks = reqs["r0"]
    trace = TT.Trace()
    trace.add([("r0", toks[:2], 0)])
    for i in range(2, len(toks)):
        trace.add([("r0", toks[i:i + 1], i)], end=["r0"] if i == len(toks) - 1 else [])
    run_trace(folder, dtype, trace, str(tmp_path), block_size=8)
    got = TT.read_logits(str(tmp_path), trace, vocab)
    TT.compare(got, ref, TOL[dtype], f"long decode/{dtype}")
    # the same again with one-token first step: position 0 alone
    trace2 = TT.Trace()
    trace2.add([("r0", toks[:1], 0)])
    trace2.add([("r0", toks[1:3], 1)])
    trace2.add([("r0", toks[3:40], 3)], end=["r0"])
    out2 = tmp_path / "first"
    run_trace(folder, dtype, trace2, str(out2), block_size=8)
    got2 = TT.read_logits(str(out2), trace2, vocab)
    TT.compare(got2, {"r0": ref["r0"][:40]}, TOL[dtype], f"first tokens/{dtype}")


def test_cut_and_batch_do_not_change_float32_logits_beyond_rounding(tmp_path):
    """All four schedules against each other (not only against the oracle)."""
    folder, vocab, reqs, _ = reference("tiny_qwen2")
    results = {}
    for schedule, make in SCHEDULES.items():
        trace = make(reqs)
        out = tmp_path / schedule
        run_trace(folder, "float32", trace, str(out), block_size=8)
        results[schedule] = TT.read_logits(str(out), trace, vocab)
    base = results["whole"]
    for schedule, got in results.items():
        for (label, pos), row in got.items():
            want = base[(label.split("#")[0], pos)]         # rows of an abandoned pass ("r0#0") are compared too
            scale = float(abs(want).max())
            assert float(abs(row - want).max()) / scale < 2e-5, f"{schedule} differs from whole at {(label, pos)}"


def test_steps_with_nothing_wanted_write_no_file(tmp_path):
    folder, vocab, reqs, _ = reference("tiny_llama")
    import json
    lines = [json.dumps({"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3], "want": []}], "end": []}),
             json.dumps({"step": 1, "entries": [{"id": "a", "tokens": [4], "want": [0]}], "end": ["a"]}),
             json.dumps({"step": 2, "entries": [], "end": []})]
    proc = subprocess.run([sys.executable, TRACE_RUN, "--model", folder, "--dtype", "bfloat16", "--out", str(tmp_path),
                           "--max-tokens", "64"], input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == ["done", "0", "done", "1", "done", "2"]
    assert sorted(os.listdir(tmp_path)) == ["1.f32"]
    assert os.path.getsize(tmp_path / "1.f32") == 4 * vocab
