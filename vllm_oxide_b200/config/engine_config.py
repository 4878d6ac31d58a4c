"""Limits fixed for an engine's lifetime.

The five knobs and their defaults are the reference's `EngineConfig`
(crates/engine/src/model.rs:37-66): max_batch_tokens 2048, max_seqs 32,
max_model_len 8192, block_size 16, kv_pool_bytes 2 GiB. Added here: the compute
dtype, an explicit page count (tests want tiny pools), the largest portion of a
prompt that one step takes, whether decode steps replay CUDA graphs, and the switches of
what makes a decode step fast (programmatic dependent launch, folded norms, running one
step ahead of the host's reads).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..errors import ConfigError

_DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32,
}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ConfigError(f"dtype {name} is not supported (bfloat16 or float32)")
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ConfigError(f"dtype {name!r} is not supported (bfloat16 or float32)") from None


@dataclass
class EngineConfig:
    max_batch_tokens: int = 2048       # most new tokens in one step, summed over requests
    max_seqs: int = 32                 # most requests in one step (= number of state slots)
    max_model_len: int = 8192          # longest prompt + output of one request
    block_size: int = 16               # tokens per cache page
    kv_pool_bytes: int = 2 << 30       # cache budget when num_pages is not given
    num_pages: Optional[int] = None    # explicit page count per cache group
    dtype: torch.dtype = torch.bfloat16
    prefill_chunk: Optional[int] = None  # most prompt tokens of one request per step
    admission_watermark_pages: int = 0   # while others run, admit a request only if so many pages stay free behind
                                         # its first portion (0: whenever a token fits)
    cuda_graphs: bool = True           # replay decode-only steps from captured graphs
    pdl: bool = True                   # programmatic dependent launch between the engine's kernels
    fold_norms: bool = True            # steps of few rows: norms and residual adds folded into the products
    pick_in_head: bool = True          # decode steps of few rows: the output head's epilogue does the pick's first pass
    step_graphs: int = 2               # other steps: record a CUDA graph when a step of the same shape class comes the
                                       # n-th time and replay it from then on (0: never; needs cuda_graphs)
    run_ahead: bool = True             # steady decode: launch step n + 1 before reading step n's tokens (needs cuda_graphs)
    device: str = "cuda:0"

    def __post_init__(self):
        self.dtype = parse_dtype(self.dtype)
        for k in ("max_batch_tokens", "max_seqs", "max_model_len", "block_size"):
            v = getattr(self, k)
            if not isinstance(v, int) or v <= 0:
                raise ConfigError(f"engine config: {k} must be a positive integer, got {v!r}")
        if self.block_size % 8 != 0:
            raise ConfigError(f"engine config: block_size must be a multiple of 8, got {self.block_size}")
        if self.num_pages is not None and self.num_pages <= 0:
            raise ConfigError("engine config: num_pages must be positive")
        if self.prefill_chunk is not None and self.prefill_chunk <= 0:
            raise ConfigError("engine config: prefill_chunk must be positive")
        if self.admission_watermark_pages < 0:
            raise ConfigError("engine config: admission_watermark_pages cannot be negative")
