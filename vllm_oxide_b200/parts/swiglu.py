"""SwiGLU feed-forward: down(silu(gate(x)) * up(x)), dense, no bias
(crates/engine/src/model.rs:325-331; activation crates/engine/src/backend/cpu/mod.rs:341-349).
gate and up are one fused matrix [Wgate; Wup], so a single product feeds the activation."""
from __future__ import annotations

import torch

from .. import kernels
from ..tuning import TUNING
from .base import FeedForward, FoldedState, StepContext, aligned
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

    def _path(self, rows: int, aligned_input: bool = True) -> str:
        """Which kernels a step of `rows` rows runs: "few" (one tcgen05 kernel, activation in its
        epilogue), "pair" (the two-SM product with the activation in its epilogue) or "separate"
        (a product to gate|up, then the activation kernel)."""
        ok = self.dtype == torch.bfloat16 and self.fused and aligned_input and self.hidden % 8 == 0
        if ok and rows <= TUNING.few_rows:
            return "few"
        if ok and rows >= TUNING.pair_gemm_from_rows:
            return "pair"
        return "separate"

    def workspace_bytes(self, rows: int) -> int:
        """The activation [rows, inter]; on the "separate" path gate|up [rows, 2 * inter] beside it.
        The largest of any step of at most `rows` rows (a step just below the row count where
        the two-SM kernel takes over needs more than one just above)."""
        es = 2 if self.dtype == torch.bfloat16 else 4

        def at(r):
            act = aligned(r * self.inter * es)
            return act + aligned(r * 2 * self.inter * es) if self._path(r) == "separate" else act
        below = TUNING.pair_gemm_from_rows - 1
        return max(at(rows), at(below)) if rows > below else at(rows)

    def folded_workspace_bytes(self, rows: int) -> int:
        return aligned(rows * self.inter * 2)

    def kernel_modules(self, dtype, max_rows):
        if dtype == torch.float32:
            return ("elementwise", "gemm_f32")
        mods = ["elementwise", "gemm_sm100"]
        if max_rows >= TUNING.pair_gemm_from_rows:
            mods.append("gemm_sm100_pair")
        return tuple(mods)

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
        path = self._path(T, kernels.gemm_sm100_supported(x, self.w_gate_up))
        if path == "few":
            # few rows: one kernel, the activation applied in the product's epilogue
            kernels.gemm_swiglu(x, self.w_gate_up, act)
        elif path == "pair":
            # many rows: the two-SM product with the activation in its epilogue (gate and up never
            # go to memory)
            kernels.gemm_pair_swiglu(x, self.w_gate_up, act)
        else:
            gate_up = matmul(x, self.w_gate_up, ctx.alloc((T, 2 * self.inter)))
            kernels.swiglu(gate_up, act)
        return matmul(act, self.w_down, out if out is not None else ctx.alloc((T, self.hidden)))
