"""How a request's tokens are picked.

The reference picks greedily only (first index of the maximum, NaN is an error:
crates/engine/src/backend/cpu/mod.rs:370-388) and stops at an optional stop token, which it keeps
in the output (crates/engine/src/generate.rs:23,105-108). Added here: temperature sampling by the
Gumbel-max rule with a per-request seed (see csrc/sampling.cu), several stop tokens, and the
capture of logits at chosen generated positions (the reference's `capture` argument,
crates/engine/src/generate.rs:46-47).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Tuple


@dataclass
class SamplingParams:
    max_new_tokens: int = 64
    temperature: float = 0.0                 # 0: greedy
    seed: int = 0                            # seed of the request's random stream
    stop_token_ids: Optional[Sequence[int]] = None   # None: the model's eos ids; (): never stop early
    capture_logits: Tuple[int, ...] = ()     # generated positions whose logits are returned

    def __post_init__(self):
        if self.max_new_tokens <= 0:
            raise ValueError("max_new_tokens must be positive")
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if self.seed < 0:
            raise ValueError("seed must be >= 0")
