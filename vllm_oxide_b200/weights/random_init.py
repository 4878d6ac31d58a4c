"""Seeded random weights: a model folder from a configuration and a seed.

The reference has random weights for its tests only (crates/engine/src/testutil.rs:34-91).
Here they are a mode of the product: each tensor of the architecture's manifest is drawn
from N(0, std) (norm weights are ones) by a generator seeded from (seed, tensor name), so a
tensor's values do not depend on which other tensors exist or in which order they are made.
`write_random_model` writes config.json and model.safetensors.
"""
from __future__ import annotations

import os
import zlib
from typing import Dict, Mapping

import torch

from ..config.model_config import write_config_json
from .loader import TensorSpec
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    return (int(seed) * 1000003 + zlib.crc32(name.encode("utf-8"))) % (1 << 62)


def random_tensors(manifest: Mapping[str, TensorSpec], seed: int, std: float = 0.02,
                   dtype: torch.dtype = torch.bfloat16, device: str = "cpu",
                   norm_jitter: float = 0.0) -> Dict[str, torch.Tensor]:
    """Draw every tensor of the manifest. `norm_jitter` > 0 makes "ones" tensors 1 + U(-j, j),
    so that a test notices a norm weight that is ignored or misapplied."""
    out = {}
    for name, spec in manifest.items():
        g = torch.Generator(device=device)
        g.manual_seed(_tensor_seed(seed, name))
        if spec.kind == "int":
            out[name] = torch.zeros(spec.shape, dtype=torch.int32, device=device)
        elif spec.init == "ones":
            t = torch.ones(spec.shape, dtype=torch.float32, device=device)
            if norm_jitter:
                t += (torch.rand(spec.shape, generator=g, device=device) * 2 - 1) * norm_jitter
            out[name] = t.to(dtype)
        elif spec.init == "zeros":
            out[name] = torch.zeros(spec.shape, dtype=dtype, device=device)
        else:
            t = torch.randn(spec.shape, generator=g, dtype=torch.float32, device=device)
            out[name] = (t * std).to(dtype)
    return out


def write_random_model(model_dir: str, config, seed: int, std: float = 0.02,
                       dtype: torch.dtype = torch.bfloat16, norm_jitter: float = 0.0) -> None:
    """Write <model_dir>/config.json and model.safetensors for `config` (any registered
    architecture's configuration object)."""
    from ..config.registry import architecture_for
    d = config.to_dict()
    arch = architecture_for(d)
    os.makedirs(model_dir, exist_ok=True)
    write_config_json(model_dir, d)
    tensors = random_tensors(arch.manifest(config), seed, std, dtype, "cpu", norm_jitter)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      {"format": "pt", "seed": str(seed), "std": str(std)})
