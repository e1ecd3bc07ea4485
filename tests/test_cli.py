"""The command line and the `rvllm` package name."""
import json
import os
import subprocess
import sys

import pytest

import tiny_configs
from model_tools import model_folder

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RVLLM = os.path.join(ROOT, "bin", "rvllm")


def run(*args, **kw):
    return subprocess.run([sys.executable, RVLLM, *args], capture_output=True, text=True, timeout=600, **kw)


def test_package_surface():
    import rvllm
    assert rvllm.__version__ == "0.1.0"
    for name in ("LLM", "SamplingParams", "Sampler", "Tokenizer"):
        assert hasattr(rvllm, name)


def test_info_and_random_weights(tmp_path):
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(tiny_configs.get("tiny_llama")))
    p = run("random-weights", "--config", str(cfg), "--out", str(tmp_path / "m"), "--seed", "5")
    assert p.returncode == 0, p.stderr
    assert sorted(os.listdir(tmp_path / "m")) == ["config.json", "model.safetensors"]
    p = run("info", "--model", str(tmp_path / "m"))
    info = json.loads(p.stdout)
    assert info["architecture"] == "LlamaForCausalLM"
    H, L, I, V = 80, 2, 172, 261
    assert info["parameters"] == 2 * V * H + L * (4 * H * H + 3 * I * H + 2 * H) + H
    assert info["kv_bytes_per_token_bf16"] == L * 2 * 5 * 16 * 2
    p = run("info", "--model", str(tmp_path / "nowhere"))
    assert p.returncode != 0 and "config.json" in p.stderr


def test_generate_refuses_what_it_cannot_run(tmp_path):
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(tiny_configs.get("tiny_llama")))
    p = run("generate", "--config", str(cfg), "--prompt-ids", "1,2")
    assert p.returncode != 0 and "--random-weights" in p.stderr
    p = run("generate", "--random-weights", "--prompt-ids", "1,2")
    assert p.returncode != 0 and "--config" in p.stderr
    p = run("generate", "--config", str(cfg), "--random-weights", "--device", "cpu", "--prompt-ids", "1,2")
    assert p.returncode != 0 and "no CPU path" in p.stderr


@pytest.mark.gpu
def test_generate_from_a_configuration_with_random_weights(tmp_path):
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(tiny_configs.get("tiny_qwen2")))
    outs = []
    for seed in ("3", "3", "4"):
        p = run("generate", "--config", str(cfg), "--random-weights", "--seed", seed, "--prompt-ids", "1,2,3",
                "--max-tokens", "6", "--ignore-eos", "--num-blocks", "32", "--max-model-len", "128", "--dtype", "float32")
        assert p.returncode == 0, p.stderr[-2000:]
        outs.append(json.loads(p.stdout.splitlines()[0])["token_ids"])
    assert outs[0] == outs[1] and len(outs[0]) == 6 and outs[0] != outs[2]


@pytest.mark.gpu
def test_generate_and_benchmark_on_the_gpu():
    folder = model_folder("tiny_llama")
    p = run("generate", "--model", folder, "--prompt-ids", "1,2,3", "--prompt-ids", "9 8 7 6", "--max-tokens", "5",
            "--ignore-eos", "--num-blocks", "32", "--max-model-len", "128")
    assert p.returncode == 0, p.stderr[-2000:]
    recs = [json.loads(l) for l in p.stdout.splitlines()]
    assert [r["prompt_tokens"] for r in recs] == [3, 4] and all(len(r["token_ids"]) == 5 for r in recs)
    env = dict(os.environ, RVLLM_MODEL_DIR=folder, RVLLM_WARMUP="2")
    p = run("benchmark", "--n", "1,4", "--input-len", "8", "--output-len", "12", "--json", "--num-blocks", "64",
            "--max-model-len", "64", env=env)
    assert p.returncode == 0, p.stderr[-2000:]
    recs = [json.loads(l) for l in p.stdout.splitlines()]
    assert [r["batch"] for r in recs] == [1, 4] and all(set(r) == {"batch", "iters", "tok_per_sec", "ms_per_step"} for r in recs)
