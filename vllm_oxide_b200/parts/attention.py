"""Causal grouped-query attention over the paged cache, as a mixer.

Per step: one fused projection to [q | k | v], rotary positions on q and k, the write of k and
v to their cache slots, attention of every row over its request's pages, the output projection
(crates/engine/src/model.rs:302-321: rmsnorm and the residual add belong to the block). The
write comes before the read, so the step's own keys are read from the cache like the older ones
(crates/engine/src/model.rs:309-311).

Parameters: head counts, head size, an optional window (the last `window` keys only), an
optional score scale (default head_dim^-1/2, crates/engine/src/backend/cpu/attention.rs:91),
and the position encoding (a `Rotary` or None). With `wk`/`wv` None the mixer writes no cache:
it must be scheduled on a cache that another layer writes.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import kernels
from ..tuning import TUNING
from .base import CacheSpec, FoldedState, LayerCache, Mixer, StepContext, aligned
from .linear import matmul, to_compute


def decode_split_rule(num_seqs: int, kv_heads: int, num_sms: int, long_context: bool = False):
    """(splits, wide): how many blocks share one request's keys in a decode step and whether they
    merge through global memory. Up to 8 blocks form a cluster and merge through shared memory:
    enough that the grid fills the GPU twice over. With long contexts and few requests (at least 4
    blocks per request and kv head at three blocks per SM, which is what fits with the three-stage
    ring), up to 64 blocks merge through global memory instead (`wide`), and a request uses as many
    of them as its length is worth. Measured with 8 kv heads of 64: one request of 131,072 keys
    175 us in clusters of 8, 51 us wide; 8 requests of 32,768 keys 107 / 94 us; below some 5,000
    keys the cluster is faster. (Merging in clusters of 8 first and only the clusters' sums through
    global memory was built and measured for one request: a decode step at batch 1 took 0.824
    instead of 0.865 ms with 8,192 keys, but 1.019 instead of 0.998 ms with 32,768, where 48 longer
    blocks per kv head replace 55. Not kept.)"""
    blocks = max(1, num_seqs * kv_heads)
    if long_context and 3 * num_sms // blocks >= 4:
        return min(64, 3 * num_sms // blocks), True
    # At least twice the SMs in blocks. One more block per request and kv head where the grid then
    # still stays within 2.6 blocks per SM and the cluster within 6 blocks (measured inside a decode
    # step, where the neighbouring kernels' blocks hold slots too: 8 requests on 8 kv heads 0.796 ms
    # a step with 6 blocks each, 0.807 with 5; but 6 requests with 8 instead of 7, or 9 with 6 instead
    # of 5, lose 5-9 %: clusters that large, or a grid that full, no longer start all at once).
    lo = -(-2 * num_sms // blocks)
    hi = (13 * num_sms // 5) // blocks
    return max(1, min(8, hi if lo < hi <= 6 else lo)), False


class Attention(Mixer):
    def __init__(self, wq: torch.Tensor, wk: Optional[torch.Tensor], wv: Optional[torch.Tensor], wo: torch.Tensor,
                 num_heads: int, num_kv_heads: int, head_dim: int, position=None, window: Optional[int] = None,
                 scale: Optional[float] = None, dtype=torch.bfloat16, device="cuda"):
        self.H, self.KV, self.hd = int(num_heads), int(num_kv_heads), int(head_dim)
        if self.H % self.KV != 0:
            raise ValueError(f"{self.H} heads are not a multiple of {self.KV} kv heads")
        if self.hd % 16 != 0 or self.hd > 256:
            raise ValueError(f"head_dim {self.hd} is not supported: multiples of 16 up to 256")
        hidden = wq.shape[1]
        if wq.shape != (self.H * self.hd, hidden) or wo.shape != (hidden, self.H * self.hd):
            raise ValueError(f"q/o projection shapes {list(wq.shape)} / {list(wo.shape)} do not fit "
                             f"{self.H} heads of {self.hd}")
        self.owns_cache = wk is not None
        if self.owns_cache:
            if wv is None or wk.shape != (self.KV * self.hd, hidden) or wv.shape != wk.shape:
                raise ValueError("k/v projection shapes do not fit the kv heads")
            # One matrix [Wq; Wk; Wv]: a single product gives q, k and v side by side. Row o of
            # the fused matrix is row o of its source, so every output element is unchanged.
            self.w_qkv = to_compute(torch.cat([wq, wk, wv], dim=0), dtype, device)
        else:
            self.w_qkv = to_compute(wq, dtype, device)
        self.w_o = to_compute(wo, dtype, device)
        self.position = position
        self.window = int(window) if window else 0
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.hd)
        self.hidden = hidden
        self.dtype = dtype
        self.impl = "auto"            # "general" forces the general attention kernel, "mma" the mma.sync kernels (tests)
        self.fused = True             # False forces the separate projection / rotary / cache-write kernels
        self.split_mixed = True       # False sends a mixed step's single tokens through the portion kernel too (tests)
        self.num_sms = torch.cuda.get_device_properties(device).multi_processor_count
        # scratch of the decode kernel's merge through global memory (one or two requests with long
        # contexts): made at the first such step, kept; the counters are zero between launches
        self._partials = None
        self._arrived = None

    def cache_spec(self) -> Optional[CacheSpec]:
        return CacheSpec(self.KV, self.hd, "window" if self.window else "full", self.window)

    def weight_bytes(self) -> int:
        return (self.w_qkv.numel() + self.w_o.numel()) * self.w_qkv.element_size()

    def _few_rows_path(self, rows: int) -> bool:
        """Steps of few rows: rotary positions and the cache write happen in the projection's epilogue."""
        return (self.dtype == torch.bfloat16 and self.fused and self.owns_cache and rows <= TUNING.few_rows
                and kernels.gemm_qkv_rope_supported(self.hd) and self.hidden % 8 == 0)

    def workspace_bytes(self, rows: int) -> int:
        """q (or q|k|v side by side) and the attention output, besides the result the block gives a place for."""
        es = 2 if self.dtype == torch.bfloat16 else 4
        q_cols = self.H * self.hd if self._few_rows_path(rows) else self.w_qkv.shape[0]
        return aligned(rows * q_cols * es) + aligned(rows * self.H * self.hd * es)

    def folded_workspace_bytes(self, rows: int) -> int:
        return 2 * aligned(rows * self.H * self.hd * 2)

    def kernel_modules(self, dtype, max_rows):
        if dtype == torch.float32:
            return ("elementwise", "gemm_f32", "attention")
        mods = ["elementwise", "gemm_sm100", "attention"]
        if self.hd in kernels.TENSOR_CORE_HEAD_DIMS:
            mods += ["attention_mma", "attention_sm100"]
        return tuple(mods)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[LayerCache], state=None, out=None) -> torch.Tensor:
        if cache is None:
            raise ValueError("attention needs a cache")
        T = x.shape[0]
        qd, kd = self.H * self.hd, self.KV * self.hd
        inv_freq = self.position.inv_freq if self.position is not None else None
        if self._few_rows_path(T) and cache.write and kernels.gemm_sm100_supported(x, self.w_qkv):
            # few rows: rotary positions and the cache write happen in the projection's epilogue
            q = ctx.alloc((T, qd))
            kernels.gemm_qkv_rope(x, self.w_qkv, q, ctx.positions, ctx.slot_mapping[cache.group], inv_freq,
                                  cache.k, cache.v, self.H, self.KV, self.hd)
            attn = ctx.alloc((T, qd))
            self.attend(q, attn, ctx, cache)
            return matmul(attn, self.w_o, out if out is not None else ctx.alloc((T, self.hidden)))
        qkv = matmul(x, self.w_qkv, ctx.alloc((T, self.w_qkv.shape[0])))
        q = qkv[:, :qd]
        if self.owns_cache and cache.write:
            k, v = qkv[:, qd:qd + kd], qkv[:, qd + kd:]
            kernels.rope_kv_write(q, k, v, ctx.positions, ctx.slot_mapping[cache.group], inv_freq,
                                  cache.k, cache.v, self.H, self.KV, self.hd)
        else:
            kernels.rope_kv_write(q, None, None, ctx.positions, None, inv_freq, None, None, self.H, self.KV, self.hd)
        attn = ctx.alloc((T, qd))
        self.attend(q, attn, ctx, cache)
        return matmul(attn, self.w_o, out if out is not None else ctx.alloc((T, self.hidden)))

    def can_fold(self) -> bool:
        """Whether this mixer can take its input in folded form (see FoldedState): bfloat16, its own
        k/v projections, a head size the fused projection epilogue takes, TMA-addressable weights."""
        return (self.dtype == torch.bfloat16 and self.fused and self.owns_cache and kernels.gemm_qkv_rope_supported(self.hd)
                and self.hidden % 8 == 0 and (self.H * self.hd) % 8 == 0)

    def forward_folded(self, st: FoldedState, eps: float, ctx: StepContext, cache: LayerCache, next_w: torch.Tensor) -> None:
        """q/k/v projection with the preceding norm folded in, rotary + cache write in its epilogue;
        attention; output projection whose epilogue adds into the residual and prepares the next
        norm's input (weight `next_w`). Updates `st` in place."""
        T = st.xn.shape[0]
        qd = self.H * self.hd
        inv_freq = self.position.inv_freq if self.position is not None else None
        q = ctx.alloc((T, qd))
        kernels.gemm_fused(st.xn, self.w_qkv, q, kernels.EPI_QKV, self.w_qkv.shape[0], ssq_in=st.ssq, eps=eps,
                           qkv=(ctx.positions, ctx.slot_mapping[cache.group] if cache.write else None, inv_freq, cache.k, cache.v,
                                self.H, self.KV, self.hd))
        attn = ctx.alloc((T, qd))
        self.attend(q, attn, ctx, cache)
        kernels.gemm_fused(attn, self.w_o, None, kernels.EPI_RESID, self.hidden, resid=(st.resid, next_w, st.xn, st.ssq))

    def attend(self, q, out, ctx: StepContext, cache: LayerCache) -> None:
        """bfloat16 with sizes the tensor-core kernels take: the decode kernel for steps of single
        tokens; for everything else the tcgen05 kernel (head size 64 or 128, no window) or the
        mma.sync portion kernel. In a mixed step the leading requests that bring one token each go
        to the decode kernel and the portions behind them to the portion kernel (a single token is
        a poor portion: one block would walk all its keys for four rows of a 128-row tile).
        Otherwise (float32, other head sizes) the general kernel."""
        page = cache.k.shape[2]
        bt = ctx.block_tables[cache.group]
        if self.dtype == torch.bfloat16 and self.impl != "general" and self.scale > 0:
            decode_ok = kernels.attn_mma_supported(self.H, self.KV, self.hd, page, True)
            if ctx.decode_only and decode_ok:
                self._attend_single(q, out, ctx, cache, bt, ctx.rows)
                return
            lead = 0
            if not ctx.decode_only and decode_ok and self.split_mixed and 0 < ctx.lead_single < ctx.seqs:
                lead = ctx.lead_single
            if (not ctx.decode_only and ctx.max_new > 0 and self.window == 0 and self.impl != "mma"
                    and kernels.attn_prefill_sm100_supported(self.H, self.KV, self.hd, page, bt.shape[1])):
                if lead:
                    self._attend_single(q, out, ctx, cache, bt, lead)
                kernels.attn_prefill_sm100(q, out, cache.k, cache.v, bt[lead:], ctx.seq_starts[lead:], ctx.context_lens[lead:],
                                           ctx.seqs - lead, ctx.max_new, self.H, self.KV, self.hd, self.scale)
                return
            if not ctx.decode_only and ctx.max_new > 0 and kernels.attn_mma_supported(self.H, self.KV, self.hd, page, False):
                if lead:
                    self._attend_single(q, out, ctx, cache, bt, lead)
                kernels.attn_prefill_mma(q, out, cache.k, cache.v, bt[lead:], ctx.seq_starts[lead:], ctx.context_lens[lead:],
                                         ctx.seqs - lead, ctx.max_new, self.H, self.KV, self.hd, self.scale, self.window)
                return
        kernels.paged_attention(q, out, cache.k, cache.v, bt, ctx.row_seq, ctx.positions, self.H, self.KV, self.hd,
                                self.scale, self.window)

    def _attend_single(self, q, out, ctx: StepContext, cache: LayerCache, bt, count: int) -> None:
        """The decode kernel on the first `count` rows, row i belonging to request i."""
        splits, wide = self.decode_splits(count, ctx.long_context)
        if wide and self._partials is None:
            floats = kernels.attn_decode_partial_floats(1, 1, self.hd, 3 * self.num_sms)    # requests x kv heads x splits <= 3 SMs
            self._partials = torch.empty(floats, dtype=torch.float32, device=q.device)
            self._arrived = torch.zeros(self.num_sms, dtype=torch.int32, device=q.device)
        kernels.attn_decode_mma(q[:count], out[:count], cache.k, cache.v, bt, ctx.positions[:count], self.H, self.KV, self.hd,
                                self.scale, self.window, splits, self._partials if wide else None, self._arrived if wide else None)

    def decode_splits(self, num_seqs: int, long_context: bool = False):
        return decode_split_rule(num_seqs, self.KV, self.num_sms, long_context)
