"""rvllm_b200: a small, whole LLM inference engine for one NVIDIA B200 (sm_100a)."""
__version__ = "0.1.0"

from .errors import (RvllmError, ConfigError, LoaderError, SchedulerError, KvExhausted, SamplingError,
                     KernelError)
from .config import (EngineConfig, LlamaConfig, Qwen2Config, load_config, config_from_dict,
                     register_architecture, known_architectures)
from .sampling import SamplingParams, Sampler
from .tokenizer import Tokenizer
from .weights import write_random_model
from .engine import LLM, Engine, StepEntry, RequestOutput, CompletionOutput

__all__ = ["LLM", "Engine", "StepEntry", "SamplingParams", "Sampler", "Tokenizer", "EngineConfig",
           "LlamaConfig", "Qwen2Config", "load_config", "config_from_dict", "register_architecture",
           "known_architectures", "write_random_model", "RequestOutput", "CompletionOutput", "RvllmError",
           "ConfigError", "LoaderError", "SchedulerError", "KvExhausted", "SamplingError", "KernelError",
           "__version__"]
