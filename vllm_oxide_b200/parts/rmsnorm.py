"""RMSNorm with the residual add folded in.

out = weight * (x * 1/sqrt(mean(x^2) + eps)), weight last, sums in float32
(crates/engine/src/backend/cpu/mod.rs:182-197). The block hands the norm the float32 residual
and the delta its previous part produced; the kernel adds the delta into the residual (the
reference's `add`, :351-358) and normalises the sum in one pass over the row.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import Norm, StepContext, aligned


class RMSNorm(Norm):
    scale_and_weight = True       # out = weight * (x * scale(x)): folds into the products around it

    def __init__(self, weight: torch.Tensor, eps: float, device):
        if weight.dim() != 1:
            raise ValueError(f"RMSNorm weight must be a vector, got {list(weight.shape)}")
        # The weight is read as float32 whatever it was stored as (widening is exact).
        self.weight = weight.to(device=device, dtype=torch.float32).contiguous()
        self.eps = float(eps)
        self.width = weight.shape[0]

    def weight_bytes(self) -> int:
        return self.weight.numel() * 4

    def workspace_bytes(self, rows: int, act_bytes: int) -> int:
        return aligned(rows * self.width * act_bytes)

    def kernel_modules(self, dtype, max_rows):
        return ("elementwise",)

    def forward(self, resid: torch.Tensor, delta: Optional[torch.Tensor], ctx: StepContext,
                rows: Optional[torch.Tensor] = None, num_rows: Optional[int] = None) -> torch.Tensor:
        n = resid.shape[0] if rows is None else (num_rows if num_rows is not None else rows.numel())
        out = ctx.alloc((n, self.width))
        kernels.add_rmsnorm(resid, delta, self.weight, self.eps, out, rows[:n] if rows is not None else None)
        return out
