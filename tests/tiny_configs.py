"""The small configurations the tests run on.  `tiny_llama` and `tiny_qwen2` differ in every
size and option; `baseline0` and `baseline1` are the two tiny configurations this project's
benchmark description names."""
from __future__ import annotations

import copy

TINY_LLAMA = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 80, "num_hidden_layers": 2, "num_attention_heads": 5, "num_key_value_heads": 5,
    "head_dim": 16, "intermediate_size": 172, "vocab_size": 261, "max_position_embeddings": 512,
    "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 32},
    "attention_bias": False, "tie_word_embeddings": False, "hidden_act": "silu", "torch_dtype": "bfloat16",
    "eos_token_id": 2,
}

TINY_QWEN2 = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "hidden_size": 96, "num_hidden_layers": 3, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 32, "intermediate_size": 200, "vocab_size": 383, "max_position_embeddings": 1024,
    "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "rope_scaling": None,
    "tie_word_embeddings": True, "hidden_act": "silu", "torch_dtype": "bfloat16",
    "use_sliding_window": True, "sliding_window": 40, "max_window_layers": 1,
    "layer_types": ["full_attention", "sliding_attention", "sliding_attention"],
    "eos_token_id": [5, 7],
}

BASELINE0 = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 172, "vocab_size": 256,
    "max_position_embeddings": 128, "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "attention_bias": False,
    "tie_word_embeddings": False, "hidden_act": "silu", "torch_dtype": "bfloat16",
}

BASELINE1 = {
    "architectures": ["Qwen2ForCausalLM"], "hidden_size": 96, "num_hidden_layers": 3, "num_attention_heads": 3,
    "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 256, "vocab_size": 384,
    "max_position_embeddings": 256, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "tie_word_embeddings": True,
    "hidden_act": "silu", "torch_dtype": "bfloat16", "use_sliding_window": False,
}

ALL = {"tiny_llama": TINY_LLAMA, "tiny_qwen2": TINY_QWEN2, "baseline0": BASELINE0, "baseline1": BASELINE1}


def get(name: str) -> dict:
    return copy.deepcopy(ALL[name])
