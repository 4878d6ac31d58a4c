"""The arrangement of parts in one layer: pre-norm residual block.

    residual += mixer(norm1(residual));  residual += feed_forward(norm2(residual))
(crates/engine/src/model.rs:302-332). The residual is float32. Each part's output is not added
at once: it is handed on as `pending` and the next norm's kernel adds it while it normalises
(one pass over the row instead of two). The model's final norm takes the last `pending`.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import FeedForward, FoldedState, LayerCache, Mixer, Norm, StepContext, aligned


class Block:
    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm, feed_forward: FeedForward):
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward

    def weight_bytes(self) -> int:
        return sum(getattr(p, "weight_bytes", lambda: 0)() for p in (self.norm1, self.mixer, self.norm2, self.feed_forward))

    def workspace_bytes(self, rows: int, hidden: int, act_bytes: int) -> int:
        """Peak scratch of one run of the block, read off the scopes of `forward`: the mixer's
        output, then the larger of (first norm's output + mixer scratch) and (second norm's output +
        feed-forward scratch)."""
        mixed = aligned(rows * hidden * act_bytes)
        return mixed + max(self.norm1.workspace_bytes(rows, act_bytes) + self.mixer.workspace_bytes(rows),
                           self.norm2.workspace_bytes(rows, act_bytes) + self.feed_forward.workspace_bytes(rows))

    def folded_workspace_bytes(self, rows: int) -> int:
        """Peak scratch of `forward_folded` (0 for parts that do not say)."""
        return max(getattr(self.mixer, "folded_workspace_bytes", lambda r: 0)(rows),
                   getattr(self.feed_forward, "folded_workspace_bytes", lambda r: 0)(rows))

    def kernel_modules(self, dtype, max_rows):
        mods = []
        for p in (self.norm1, self.mixer, self.norm2, self.feed_forward):
            mods += list(getattr(p, "kernel_modules", lambda d, r: ())(dtype, max_rows))
        return tuple(mods)

    def can_fold(self) -> bool:
        """Whether this block can run in folded form (see FoldedState): both norms are a per-token
        scale and a per-feature weight (`Norm.scale_and_weight`), which is what folds into the
        neighbouring products, and mixer and feed-forward both offer it."""
        return (self.norm1.scale_and_weight and self.norm2.scale_and_weight
                and getattr(self.mixer, "can_fold", lambda: False)() and getattr(self.feed_forward, "can_fold", lambda: False)()
                and self.mixer.state_spec() is None)

    def forward_folded(self, st: FoldedState, ctx: StepContext, cache: Optional[LayerCache], next_norm: Norm) -> None:
        """The block on the folded residual: no norm kernel, no separate residual add. `next_norm`
        is the norm that will read the residual after this block (the next block's first norm, or
        the model's final norm)."""
        with ctx.workspace.scope():
            self.mixer.forward_folded(st, self.norm1.eps, ctx, cache, self.norm2.weight)
        with ctx.workspace.scope():
            self.feed_forward.forward_folded(st, self.norm2.eps, ctx, next_norm.weight)

    def forward(self, resid: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                cache: Optional[LayerCache], state: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
        """Runs the block. `pending` is the previous block's output that is still to be added to
        the residual; the feed-forward's output (again not yet added) is written to `out`,
        which outlives the block's own scratch."""
        ws = ctx.workspace
        with ws.scope():
            mixed = ctx.alloc(out.shape, out.dtype)
            with ws.scope():
                normed = self.norm1.forward(resid, pending, ctx)
                m = self.mixer.forward(normed, ctx, cache, state, out=mixed)
                if m.data_ptr() != mixed.data_ptr():
                    mixed.copy_(m)
            normed2 = self.norm2.forward(resid, mixed, ctx)
            ff = self.feed_forward.forward(normed2, ctx, out=out)
            if ff.data_ptr() != out.data_ptr():
                out.copy_(ff)
        return out
