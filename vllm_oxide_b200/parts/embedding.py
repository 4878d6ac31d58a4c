"""Token embedding (row gather into the float32 residual, crates/engine/src/backend/cpu/mod.rs:172-180)
and the output head (logits = normed x E^T in float32; E is the embedding table when the
configuration ties them, crates/engine/src/model.rs:344)."""
from __future__ import annotations

import torch

from .. import kernels
from ..tuning import TUNING
from .base import FoldedState, StepContext
from .linear import to_compute


class Embedding:
    def __init__(self, table: torch.Tensor, dtype=torch.bfloat16, device="cuda"):
        self.table = to_compute(table, dtype, device)
        self.vocab, self.hidden = self.table.shape
        self.err_flag = torch.zeros(1, dtype=torch.int32, device=device)

    def kernel_modules(self, dtype, max_rows):
        return ("elementwise",)

    def forward(self, ctx: StepContext) -> torch.Tensor:
        resid = ctx.alloc((ctx.rows, self.hidden), torch.float32)
        kernels.embed(self.table, ctx.tokens, resid, self.err_flag)
        return resid

    def forward_folded(self, ctx: StepContext, next_norm) -> FoldedState:
        """The embedding with the first norm's input prepared (see FoldedState)."""
        h = self.hidden
        st = FoldedState(resid=ctx.alloc((ctx.rows, h), torch.float32), xn=ctx.alloc((ctx.rows, h), torch.bfloat16),
                         ssq=ctx.alloc((-(-h // 128), TUNING.few_rows), torch.float32))
        kernels.embed_fold(self.table, ctx.tokens, st.resid, next_norm.weight, st.xn, st.ssq, self.err_flag)
        return st


class LMHead:
    """`weight` may be the Embedding's own table (tied): no copy is made then."""

    def __init__(self, weight: torch.Tensor):
        self.weight = weight
        self.vocab, self.hidden = weight.shape

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def kernel_modules(self, dtype, max_rows):
        return ("gemm_f32",) if dtype == torch.float32 else ("gemm_sm100",)

    def forward(self, normed: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        kernels.linear(normed, self.weight, out)
        return out

    def can_fold(self) -> bool:
        return self.weight.dtype == torch.bfloat16 and self.hidden % 8 == 0

    def forward_folded(self, st: FoldedState, eps: float, rows: int, out: torch.Tensor) -> torch.Tensor:
        """Logits of the first `rows` rows straight from the folded residual: the final norm is the
        per-token scale of the product."""
        kernels.gemm_fused(st.xn[:rows], self.weight, out, kernels.EPI_STORE, self.vocab, ssq_in=st.ssq, eps=eps)
        return out

    def pick_folded(self, st: FoldedState, eps: float, rows: int, temperature, seeds, steps, part_val: torch.Tensor,
                    part_idx: torch.Tensor, nan_flags: torch.Tensor, out: torch.Tensor, also=()) -> None:
        """Tokens of the first `rows` rows straight from the folded residual, without the logits ever
        going to memory: the head product's epilogue leaves the best (value, index) pair of every
        128 logits, a second small kernel reduces a row's pairs. Same picks as `forward_folded`
        followed by `kernels.pick_tokens` (the same values, compared by the same rule). `also`: further
        places the tokens are written to (see `kernels.pick_final`)."""
        kernels.gemm_fused(st.xn[:rows], self.weight, None, kernels.EPI_PICK, self.vocab, ssq_in=st.ssq, eps=eps,
                           pick=(temperature, seeds, steps, part_val, part_idx, nan_flags))
        kernels.pick_final(part_val, part_idx, rows, self.vocab, nan_flags, out, also)
