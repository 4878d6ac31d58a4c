"""SwiGLU feed-forward: down(silu(gate(x)) * up(x)), dense, no bias
(crates/engine/src/model.rs:325-331; activation crates/engine/src/backend/cpu/mod.rs:341-349).
gate and up are one fused matrix [Wgate; Wup], so a single product feeds the activation."""
from __future__ import annotations

import torch

from .. import kernels
from .base import FeedForward, FoldedState, StepContext
from .linear import matmul, to_compute


class SwiGLU(FeedForward):
    def __init__(self, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, dtype=torch.bfloat16, device="cuda"):
        inter, hidden = w_gate.shape
        if w_up.shape != (inter, hidden) or w_down.shape != (hidden, inter):
            raise ValueError(f"feed-forward shapes do not fit: gate {list(w_gate.shape)}, up {list(w_up.shape)}, "
                             f"down {list(w_down.shape)}")
        self.inter, self.hidden = inter, hidden
        self.w_gate_up = to_compute(torch.cat([w_gate, w_up], dim=0), dtype, device)
        self.w_down = to_compute(w_down, dtype, device)
        self.dtype = dtype
        self.fused = True             # False forces the separate product + activation kernels (tests)

    def weight_bytes(self) -> int:
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def workspace_bytes(self, rows: int) -> int:
        es = 2 if self.dtype == torch.bfloat16 else 4
        return rows * 3 * self.inter * es + 2 * 256

    def can_fold(self) -> bool:
        return self.dtype == torch.bfloat16 and self.fused and self.hidden % 8 == 0 and self.inter % 8 == 0

    def forward_folded(self, st: FoldedState, eps: float, ctx: StepContext, next_w: torch.Tensor) -> None:
        """gate/up product with the preceding norm folded in and the activation in its epilogue;
        down product whose epilogue adds into the residual and prepares the next norm's input."""
        T = st.xn.shape[0]
        act = ctx.alloc((T, self.inter))
        kernels.gemm_fused(st.xn, self.w_gate_up, act, kernels.EPI_SWIGLU, self.inter, ssq_in=st.ssq, eps=eps)
        kernels.gemm_fused(act, self.w_down, None, kernels.EPI_RESID, self.hidden, resid=(st.resid, next_w, st.xn, st.ssq))

    def forward(self, x: torch.Tensor, ctx: StepContext, out=None) -> torch.Tensor:
        T = x.shape[0]
        act = ctx.alloc((T, self.inter))
        if (self.dtype == torch.bfloat16 and T <= kernels.FUSED_GEMM_BEST_ROWS and self.fused
                and kernels.gemm_sm100_supported(x, self.w_gate_up)):
            # few rows: one kernel, the activation applied in the product's epilogue
            kernels.gemm_swiglu(x, self.w_gate_up, act)
        elif (self.dtype == torch.bfloat16 and T >= kernels.PAIR_GEMM_FROM_ROWS and self.fused
                and kernels.gemm_sm100_supported(x, self.w_gate_up)):
            # many rows: the two-SM product with the activation in its epilogue (gate and up never
            # go to memory)
            kernels.gemm_pair_swiglu(x, self.w_gate_up, act)
        else:
            gate_up = matmul(x, self.w_gate_up, ctx.alloc((T, 2 * self.inter)))
            kernels.swiglu(gate_up, act)
        return matmul(act, self.w_down, out if out is not None else ctx.alloc((T, self.hidden)))
