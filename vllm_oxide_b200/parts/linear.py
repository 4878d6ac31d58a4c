"""A weight matrix [out, in] in the compute dtype and its product with activations."""
from __future__ import annotations

import torch

from .. import kernels


def to_compute(w: torch.Tensor, dtype: torch.dtype, device) -> torch.Tensor:
    """Move a stored tensor to the device in the compute dtype. bfloat16 -> float32 is exact
    (crates/engine/src/weights.rs:93-95); float32 -> bfloat16 rounds to nearest even."""
    return w.to(device=device, dtype=dtype).contiguous()


def matmul(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    kernels.linear(x, w, out)
    return out
