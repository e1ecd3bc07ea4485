"""Weights: safetensors reading and writing, binding by name, one error for everything wrong,
and the random-weights mode."""
import json
import os
import struct

import pytest
import torch

import tiny_configs
from rvllm_b200 import LoaderError, config_from_dict, write_random_model
from rvllm_b200.models import DecoderModel, expected_tensors
from rvllm_b200.weights import SafetensorsFile, WeightSource, engine_dtype_of, write_safetensors
from rvllm_b200.weights.safetensors_io import open_model_files


def test_round_trip_and_agreement_with_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file, save_file
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).bfloat16(), "c": torch.arange(6, dtype=torch.int32).view(2, 3),
         "d": torch.randn(2, 2).half()}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t, {"k": "v"})
    theirs = load_file(p)                      # our writer, their reader
    for k in t:
        assert torch.equal(theirs[k], t[k])
    f = SafetensorsFile(p)                     # our writer, our reader
    assert f.metadata == {"k": "v"}
    for k in t:
        assert torch.equal(f.tensor(k), t[k]) and f.tensor(k).dtype == t[k].dtype
    p2 = str(tmp_path / "y.safetensors")
    save_file(t, p2)                           # their writer, our reader
    f2 = SafetensorsFile(p2)
    for k in t:
        assert torch.equal(f2.tensor(k), t[k])


def _raw(tmp_path, header: dict, data: bytes, name="bad.safetensors", hlen=None):
    blob = json.dumps(header).encode()
    p = tmp_path / name
    p.write_bytes(struct.pack("<Q", len(blob) if hlen is None else hlen) + blob + data)
    return str(p)


def test_corrupt_files_are_refused(tmp_path):
    (tmp_path / "short.safetensors").write_bytes(b"\x01\x02")
    with pytest.raises(LoaderError, match="too short"):
        SafetensorsFile(str(tmp_path / "short.safetensors"))
    with pytest.raises(LoaderError, match="exceeds the file"):
        SafetensorsFile(_raw(tmp_path, {}, b"", hlen=10 ** 9))
    p = tmp_path / "nojson.safetensors"
    p.write_bytes(struct.pack("<Q", 4) + b"{{{{")
    with pytest.raises(LoaderError, match="JSON"):
        SafetensorsFile(str(p))
    with pytest.raises(LoaderError, match="unsupported dtype"):
        SafetensorsFile(_raw(tmp_path, {"w": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}, b"0000"))
    with pytest.raises(LoaderError, match="dtype\\*shape"):
        SafetensorsFile(_raw(tmp_path, {"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}, b"0" * 16))
    with pytest.raises(LoaderError, match="beyond the file"):
        SafetensorsFile(_raw(tmp_path, {"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}, b"0" * 8))
    with pytest.raises(LoaderError, match="neither"):
        open_model_files(str(tmp_path / "empty"))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = config_from_dict(tiny_configs.get("tiny_llama"))
    d = write_random_model(cfg, str(tmp_path / "m"), seed=0)
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    tensors = {k: f.tensor(k).clone() for k in f.entries}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(80)
    tensors["lm_head.weight"] = torch.zeros(261, 81)
    tensors["model.layers.0.input_layernorm.weight"] = torch.zeros(79)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    src = WeightSource(d)
    expected = {n: ts.shape for n, ts in expected_tensors(cfg.to_spec()).items()}
    with pytest.raises(LoaderError) as e:
        src.check(expected, cfg.to_spec().ignored_tensors)
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert len(err.wrong_shape) == 2 and "lm_head.weight" in err.wrong_shape[0] and "[261, 81]" in err.wrong_shape[0]
    msg = str(err)
    for part in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (2)", "up_proj", "q_proj.bias"):
        assert part in msg


def test_expected_names_follow_the_checkpoint_convention():
    q = expected_tensors(config_from_dict(tiny_configs.get("tiny_qwen2")).to_spec())
    assert "lm_head.weight" not in q                       # tied: the embedding is the LM head
    assert q["model.layers.2.self_attn.k_proj.bias"].shape == (64,)
    assert q["model.layers.0.mlp.gate_proj.weight"].shape == (200, 96)
    assert q["model.embed_tokens.weight"].shape == (383, 96)
    l = expected_tensors(config_from_dict(tiny_configs.get("tiny_llama")).to_spec())
    assert l["lm_head.weight"].shape == (261, 80) and not any("bias" in n for n in l)
    assert l["model.layers.1.post_attention_layernorm.weight"].init == "norm"


def test_ignored_tensors_and_shards(tmp_path):
    cfg = config_from_dict(tiny_configs.get("tiny_llama"))
    d = write_random_model(cfg, str(tmp_path / "m"), seed=1)
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    tensors = {k: f.tensor(k).clone() for k in f.entries}
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    names = sorted(tensors)
    half = len(names) // 2
    os.remove(os.path.join(d, "model.safetensors"))
    write_safetensors(os.path.join(d, "model-00001-of-00002.safetensors"), {n: tensors[n] for n in names[:half]})
    write_safetensors(os.path.join(d, "model-00002-of-00002.safetensors"), {n: tensors[n] for n in names[half:]})
    index = {"weight_map": {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
                            for i, n in enumerate(names)}}
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as fh:
        json.dump(index, fh)
    src = WeightSource(d)
    expected = {n: ts.shape for n, ts in expected_tensors(cfg.to_spec()).items()}
    src.check(expected, cfg.to_spec().ignored_tensors)      # inv_freq is skipped, both shards are read
    got = src.get("model.norm.weight", torch.bfloat16, "cpu")
    assert torch.equal(got, tensors["model.norm.weight"])


def test_dtype_rule():
    bf, f32 = torch.bfloat16, torch.float32
    assert engine_dtype_of(torch.bfloat16, bf) == bf
    assert engine_dtype_of(torch.float16, bf) == bf
    assert engine_dtype_of(torch.float32, bf) == f32         # stored in 32 bits: stays so
    assert engine_dtype_of(torch.bfloat16, f32) == f32
    assert engine_dtype_of(torch.int64, bf) == torch.int32   # integer tables


def test_random_weights_are_reproducible_and_distributed_as_stated(tmp_path):
    cfg = config_from_dict(tiny_configs.get("tiny_qwen2"))
    a = write_random_model(cfg, str(tmp_path / "a"), seed=7)
    b = write_random_model(cfg, str(tmp_path / "b"), seed=7)
    c = write_random_model(cfg, str(tmp_path / "c"), seed=8)
    fa, fb, fc = (SafetensorsFile(os.path.join(x, "model.safetensors")) for x in (a, b, c))
    assert set(fa.entries) == set(expected_tensors(cfg.to_spec()))
    for k in fa.entries:
        assert torch.equal(fa.tensor(k), fb.tensor(k))
    assert not torch.equal(fa.tensor("model.embed_tokens.weight"), fc.tensor("model.embed_tokens.weight"))
    w = fa.tensor("model.embed_tokens.weight").float()
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    g = torch.cat([fa.tensor(f"model.layers.{i}.input_layernorm.weight").float() for i in range(3)])
    assert abs(float(g.mean()) - 1.0) < 0.05 and abs(float(g.std()) - 0.1) < 0.03
    with open(os.path.join(a, "config.json")) as fh:
        assert config_from_dict(json.load(fh)) == cfg


def test_model_binds_and_fuses_by_name(tmp_path):
    cfg = config_from_dict(tiny_configs.get("tiny_qwen2"))
    d = write_random_model(cfg, str(tmp_path / "m"), seed=3)
    src = WeightSource(d)
    model = DecoderModel(cfg.to_spec())
    model.load(lambda n: src.get(n, torch.float32, "cpu"), torch.float32, "cpu", 64)
    att = model.layers[1].mixer
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    q, k, v = (f.tensor(f"model.layers.1.self_attn.{n}_proj.weight").float() for n in "qkv")
    assert torch.equal(att.qkv.weight, torch.cat([q, k, v]))
    assert att.qkv.bias.shape == (6 * 32 + 2 * 2 * 32,)
    assert model.lm_head is model.embedding                  # tied
    assert model.position_encodings["rope"].cos.shape == (64, 16)
