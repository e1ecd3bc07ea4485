"""Options of the engine (not of the model), validated all at once.

After the reference's `RuntimeConfig` and its validating builder
(v3/crates/rvllm-core/src/config/runtime.rs:7-44, config/builder.rs:61-142) and the option
names of its server (v3/crates/rvllm-serve/src/lib.rs:47-78): `max_model_len`,
`max_num_seqs`, `max_num_batched_tokens`, `max_prefill_chunk`, `gpu_memory_utilization`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from ..errors import ConfigError

_DTYPES = {"bfloat16": "bfloat16", "bf16": "bfloat16", "float32": "float32", "fp32": "float32",
           "f32": "float32"}


def canonical_dtype(name: str) -> str:
    if name not in _DTYPES:
        raise ConfigError(f"dtype {name!r} is not supported (known: bfloat16, float32)")
    return _DTYPES[name]


@dataclass(frozen=True)
class EngineConfig:
    dtype: str = "bfloat16"                 # "bfloat16": serving kernels; "float32": true 32-bit
    block_size: int = 16                    # tokens per cache page
    num_blocks: Optional[int] = None        # pages per cache group; None: from memory
    gpu_memory_utilization: float = 0.9
    max_model_len: Optional[int] = None     # None: the model's max_position_embeddings
    max_num_seqs: int = 64
    max_num_batched_tokens: int = 2048
    max_prefill_chunk: Optional[int] = None  # None: limited by the token budget only
    enable_chunked_prefill: bool = True
    enforce_eager: bool = False             # never replay decode steps from CUDA graphs
    cuda_graph_batch_sizes: Tuple[int, ...] = (1, 2, 4, 8, 16, 32, 64)
    seed: int = 0
    device: str = "cuda:0"

    def validated(self, max_position_embeddings: int) -> "EngineConfig":
        """Return a copy with defaults filled in, or raise one error naming every problem."""
        p = []
        dtype = self.dtype
        if dtype not in _DTYPES:
            p.append(f"dtype {dtype!r} is not supported (known: bfloat16, float32)")
        else:
            dtype = _DTYPES[dtype]
        if self.block_size < 1 or self.block_size > 256 or (self.block_size & (self.block_size - 1)):
            p.append(f"block_size must be a power of two in [1, 256], got {self.block_size}")
        if self.num_blocks is not None and self.num_blocks < 1:
            p.append(f"num_blocks must be >= 1, got {self.num_blocks}")
        if not 0.0 < self.gpu_memory_utilization <= 0.98:
            p.append(f"gpu_memory_utilization must be in (0, 0.98], got {self.gpu_memory_utilization}")
        mml = self.max_model_len if self.max_model_len is not None else max_position_embeddings
        if mml < 1:
            p.append(f"max_model_len must be >= 1, got {mml}")
        if mml > max_position_embeddings:
            p.append(f"max_model_len {mml} exceeds the model's max_position_embeddings {max_position_embeddings}")
        if self.max_num_seqs < 1:
            p.append(f"max_num_seqs must be >= 1, got {self.max_num_seqs}")
        if self.max_num_batched_tokens < 1:
            p.append(f"max_num_batched_tokens must be >= 1, got {self.max_num_batched_tokens}")
        if self.max_num_batched_tokens < self.max_num_seqs:
            p.append(f"max_num_batched_tokens {self.max_num_batched_tokens} is smaller than max_num_seqs "
                     f"{self.max_num_seqs}: a step could not decode every running request")
        if self.max_prefill_chunk is not None and self.max_prefill_chunk < 1:
            p.append(f"max_prefill_chunk must be >= 1, got {self.max_prefill_chunk}")
        if not self.enable_chunked_prefill and mml > self.max_num_batched_tokens:
            p.append(f"without chunked prefill a prompt of max_model_len {mml} tokens cannot fit "
                     f"max_num_batched_tokens {self.max_num_batched_tokens}")
        if any(b < 1 for b in self.cuda_graph_batch_sizes):
            p.append(f"cuda_graph_batch_sizes must be positive, got {self.cuda_graph_batch_sizes}")
        if p:
            raise ConfigError(p, "engine options")
        from dataclasses import replace
        return replace(self, dtype=dtype, max_model_len=mml,
                       cuda_graph_batch_sizes=tuple(sorted(set(self.cuda_graph_batch_sizes))))
