from .spec import PartSpec, LayerSpec, RunEntry, ModelSpec, default_run_order, mixer, feed_forward, norm
from .model_config import DenseDecoderConfig, LlamaConfig, Qwen2Config, RopeScaling, read_config_json
from .registry import (register_architecture, unregister_architecture, known_architectures,
                       config_from_dict, load_config)
from .engine_config import EngineConfig, canonical_dtype
