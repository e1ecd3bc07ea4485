"""Configuration: typed reading of config.json keys, the registry, engine options."""
import copy
import json
import os

import pytest

import tiny_configs
from rvllm_b200 import ConfigError, EngineConfig, LlamaConfig, Qwen2Config, config_from_dict, load_config
from rvllm_b200.config import known_architectures, register_architecture, unregister_architecture


def test_reads_every_key_of_both_architectures():
    a = config_from_dict(tiny_configs.get("tiny_llama"))
    b = config_from_dict(tiny_configs.get("tiny_qwen2"))
    assert isinstance(a, LlamaConfig) and isinstance(b, Qwen2Config)
    assert (a.hidden_size, a.num_hidden_layers, a.num_attention_heads, a.num_key_value_heads) == (80, 2, 5, 5)
    assert (a.head_dim, a.intermediate_size, a.vocab_size, a.rms_norm_eps) == (16, 172, 261, 1e-5)
    assert a.rope_scaling.factor == 8.0 and a.rope_scaling.original_max_position_embeddings == 32
    assert not a.attention_bias and not a.tie_word_embeddings and a.eos_token_ids == (2,)
    assert a.layer_windows == (None, None)
    assert (b.hidden_size, b.num_hidden_layers, b.num_attention_heads, b.num_key_value_heads) == (96, 3, 6, 2)
    assert b.attention_bias and b.tie_word_embeddings and b.rope_theta == 1e6 and b.rope_scaling is None
    assert b.layer_windows == (None, 40, 40) and b.eos_token_ids == (5, 7)


def test_the_two_tiny_configurations_differ_in_every_size_and_option():
    a = config_from_dict(tiny_configs.get("tiny_llama"))
    b = config_from_dict(tiny_configs.get("tiny_qwen2"))
    for f in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
              "intermediate_size", "vocab_size", "max_position_embeddings", "rms_norm_eps", "rope_theta",
              "rope_scaling", "attention_bias", "tie_word_embeddings", "layer_windows"):
        assert getattr(a, f) != getattr(b, f), f
    assert a.num_attention_heads // a.num_key_value_heads != b.num_attention_heads // b.num_key_value_heads
    for v in (a.hidden_size, a.vocab_size, a.intermediate_size, b.vocab_size, b.intermediate_size):
        assert v & (v - 1), "sizes that are no power of two"


def test_defaults():
    d = tiny_configs.get("baseline0")
    del d["num_key_value_heads"], d["head_dim"], d["rope_theta"]
    c = config_from_dict(d)
    assert c.num_key_value_heads == c.num_attention_heads == 4
    assert c.head_dim == 16 and c.rope_theta == 10000.0
    q = tiny_configs.get("baseline1")
    assert config_from_dict(q).attention_bias is True          # Qwen2: bias on q, k, v without a key for it


def test_all_problems_are_reported_together():
    d = tiny_configs.get("tiny_llama")
    del d["hidden_size"], d["rms_norm_eps"]
    d["vocab_size"] = "many"
    d["hidden_act"] = "gelu"
    d["num_key_value_heads"] = 3
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    msg = str(e.value)
    for part in ("hidden_size", "rms_norm_eps", "vocab_size", "hidden_act", "num_key_value_heads"):
        assert part in msg
    assert len(e.value.reasons) >= 5


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size",
                                 "vocab_size", "max_position_embeddings", "rms_norm_eps"])
def test_each_required_key(key):
    d = tiny_configs.get("tiny_qwen2")
    del d[key]
    with pytest.raises(ConfigError, match=key):
        config_from_dict(d)


def test_unknown_architecture_lists_known_ones():
    d = tiny_configs.get("tiny_llama")
    d["architectures"] = ["MambaForCausalLM"]
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert "LlamaForCausalLM" in str(e.value) and "Qwen2ForCausalLM" in str(e.value)
    with pytest.raises(ConfigError):
        config_from_dict({"hidden_size": 8})


def test_unsupported_options_are_refused():
    d = tiny_configs.get("tiny_llama")
    d["rope_scaling"] = {"rope_type": "yarn", "factor": 2.0}
    with pytest.raises(ConfigError, match="yarn"):
        config_from_dict(d)
    d = tiny_configs.get("tiny_llama")
    d["sliding_window"] = 16
    with pytest.raises(ConfigError, match="sliding_window"):
        config_from_dict(d)
    d = tiny_configs.get("tiny_qwen2")
    d["layer_types"] = ["full_attention", "linear_attention", "full_attention"]
    with pytest.raises(ConfigError, match="linear_attention"):
        config_from_dict(d)
    d = tiny_configs.get("tiny_qwen2")
    d["attention_bias"] = False
    with pytest.raises(ConfigError, match="attention_bias"):
        config_from_dict(d)


def test_window_layers_from_max_window_layers():
    d = tiny_configs.get("tiny_qwen2")
    del d["layer_types"]
    d["max_window_layers"] = 2
    assert config_from_dict(d).layer_windows == (None, None, 40)
    d["use_sliding_window"] = False
    assert config_from_dict(d).layer_windows == (None, None, None)


def test_config_json_round_trip(tmp_path):
    for name in tiny_configs.ALL:
        c = config_from_dict(tiny_configs.get(name))
        (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
        assert load_config(str(tmp_path)) == c
    (tmp_path / "config.json").write_text("{ not json")
    with pytest.raises(ConfigError, match="JSON"):
        load_config(str(tmp_path))
    with pytest.raises(ConfigError, match="config.json"):
        load_config(str(tmp_path / "nowhere"))


def test_spec_carries_the_sizes_layer_by_layer():
    spec = config_from_dict(tiny_configs.get("tiny_qwen2")).to_spec()
    assert [l.parts["mixer"].params["window"] for l in spec.layers] == [None, 40, 40]
    assert all(l.parts["mixer"].params["qkv_bias"] for l in spec.layers)
    assert spec.lm_head_name is None and spec.layers[1].prefix == "model.layers.1."
    assert [(e.layer, e.cache) for e in spec.run_order] == [(0, 0), (1, 1), (2, 2)]
    assert spec.layers[0].parts["mixer_norm"].params == {"size": 96, "eps": 1e-6}


def test_registry_accepts_new_architectures():
    class Toy:
        @classmethod
        def from_dict(cls, obj, where=""):
            return cls()

        def to_spec(self):
            return None

    register_architecture("ToyForCausalLM", Toy)
    try:
        assert "ToyForCausalLM" in known_architectures()
        assert isinstance(config_from_dict({"architectures": ["ToyForCausalLM"]}), Toy)
    finally:
        unregister_architecture("ToyForCausalLM")
    with pytest.raises(TypeError):
        register_architecture("Broken", object)


def test_engine_options_are_validated_together():
    with pytest.raises(ConfigError) as e:
        EngineConfig(dtype="fp8", block_size=12, max_num_seqs=0, gpu_memory_utilization=1.5,
                     max_model_len=4096).validated(max_position_embeddings=1024)
    assert len(e.value.reasons) >= 5
    ok = EngineConfig(dtype="bf16", max_model_len=None).validated(512)
    assert ok.dtype == "bfloat16" and ok.max_model_len == 512


def test_llama_attention_bias_reaches_the_output_projection_and_mlp_bias_is_refused():
    from rvllm_b200.models.decoder import expected_tensors
    d = tiny_configs.get("baseline0")
    d["attention_bias"] = True
    names = expected_tensors(config_from_dict(d).to_spec())
    for proj in ("q_proj", "k_proj", "v_proj", "o_proj"):
        assert f"model.layers.1.self_attn.{proj}.bias" in names
    assert not any("mlp" in n and n.endswith(".bias") for n in names)
    q = expected_tensors(config_from_dict(tiny_configs.get("baseline1")).to_spec())
    assert "model.layers.0.self_attn.q_proj.bias" in q and "model.layers.0.self_attn.o_proj.bias" not in q
    d["mlp_bias"] = True
    with pytest.raises(ConfigError, match="mlp_bias"):
        config_from_dict(d)
