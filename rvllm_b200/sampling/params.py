"""Per-request sampling parameters.

Fields as the reference's `SamplingParams {temperature, top_k, top_p, seed}`
(v3/crates/rvllm-sampling/src/params.rs:7-28): temperature 0 is greedy.  `max_tokens`,
`stop_token_ids` and `ignore_eos` are what its evaluation loop takes from the environment
(RVLLM_MAX_TOKENS default 256, RVLLM_EOS; v3/crates/rvllm-bench/src/bin/rvllm_eval.rs:83-86,
624-629).

What the filters keep (the reference defines `top_k` and `top_p` as fields only and samples
greedily, so the rule is this project's): both act on softmax(logits / temperature) of the whole
vocabulary.  `top_k` keeps the k most likely tokens, `top_p` the smallest set of most likely tokens
whose probability reaches top_p, in both cases with every token as likely as the last kept one.
With both set, a token is kept if BOTH keep it: the top-p mass is counted on the whole
distribution, not on the one renormalised after top-k (libraries that apply the filters one after
the other keep fewer tokens when k cuts off much mass).  The draw is then made from the kept
tokens, renormalised, by inverse CDF in vocabulary order.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

from ..errors import SamplingError


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0                 # 0: off
    top_p: float = 1.0             # 1: off
    seed: Optional[int] = None     # None: derived from the engine's seed and the request's number
    max_tokens: int = 16
    stop_token_ids: Tuple[int, ...] = ()
    ignore_eos: bool = False

    def __post_init__(self):
        problems = []
        if not (self.temperature >= 0.0):
            problems.append(f"temperature must be >= 0, got {self.temperature}")
        if self.top_k < 0:
            problems.append(f"top_k must be >= 0 (0 switches it off), got {self.top_k}")
        if not (0.0 < self.top_p <= 1.0):
            problems.append(f"top_p must be in (0, 1], got {self.top_p}")
        if self.max_tokens < 1:
            problems.append(f"max_tokens must be >= 1, got {self.max_tokens}")
        if self.seed is not None and not (0 <= self.seed < 2 ** 63):
            problems.append(f"seed must be in [0, 2^63), got {self.seed}")
        if problems:
            raise SamplingError("; ".join(problems))
        object.__setattr__(self, "stop_token_ids", tuple(self.stop_token_ids))

    @property
    def is_greedy(self) -> bool:
        return self.temperature == 0.0

    @staticmethod
    def greedy(max_tokens: int = 16) -> "SamplingParams":
        return SamplingParams(temperature=0.0, max_tokens=max_tokens)
