"""The step function: one batch of (request, its next tokens) through the model, from the cache.

The reference has two entry points, prefill and decode, and a step is all one or all the other
(crates/engine/src/model.rs:221-243); its attention, though, is one function fed the same
per-row arrays in both (crates/engine/src/backend/cpu/mod.rs:310,337), and a decode row is a
portion of length one. So here there is ONE `step`: any mix of portions of prompts and single
decoded tokens runs as one batch, reads older keys from the cache, writes its own, and returns
the logits at the wanted places together with a token picked from each.

Order inside a layer is the reference's (crates/engine/src/model.rs:302-332): norm, q/k/v,
rotary, cache write, attention, output projection + residual, norm, gate/up, SwiGLU, down +
residual; then the final norm and the head on the wanted rows only (:335-344).
"""
from __future__ import annotations

import collections
import os
import sys
from dataclasses import dataclass
from typing import List, Optional

import torch

from .. import kernels
from ..cache.pools import CachePools
from ..config import EngineConfig, architecture_for, read_config_json
from ..csrc.build import runtime_module
from ..errors import CapacityError, KernelError, ShapeError
from ..tuning import TUNING
from ..parts.base import ModelSpec, StepContext, Workspace, aligned
from ..weights import load_safetensors_weights, weights_from_tensors


@dataclass
class StepResult:
    sampled: torch.Tensor                 # int32 [R] on the device: the token picked at each wanted row
    logits: Optional[torch.Tensor]        # float32 [R, vocab] where the caller asked for them
    num_logit_rows: int

    def tokens(self) -> List[int]:
        """The picked tokens on the host (this is the step's one device-to-host read)."""
        return self.sampled[:self.num_logit_rows].tolist()


def step_shape_class(rows: int, seqs: int, logit_count: int, max_new: int, lead_single: int, max_seq_len: int,
                     rows_cap: int):
    """The shape class under which a step that is no decode step is recorded and replayed:
    (rows rounded up to 16 / 32 / 64 / a multiple of 128, never beyond `rows_cap`; requests; wanted
    rows; the longest portion rounded up to 64, never beyond the rows; leading single tokens; long
    contexts or not). None for a decode step and for a step that wants no logits."""
    if logit_count == 0 or (max_new == 1 and rows == seqs):
        return None
    padded = min(16 if rows <= 16 else 32 if rows <= 32 else 64 if rows <= 64 else -(-rows // 128) * 128, rows_cap)
    longest = min(-(-max_new // 64) * 64, padded)
    return (padded, seqs, logit_count, longest, int(lead_single), bool(max_seq_len > TUNING.long_context_keys))


def _require_cuda(device: str) -> None:
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device is available; this engine has no CPU path")
    if not str(device).startswith("cuda"):
        raise KernelError(f"device {device!r}: this engine runs on a CUDA device only")


def decode_bucket(n: int) -> int:
    """The batch-size class a decode step of `n` requests is recorded under: 1, 2, 3, 4, 6, 8, 12, 16,
    24, 32, ... (powers of two and the sizes half way between: a step of 9 requests padded to 16 would
    share its keys over blocks as 16 requests do, 0.90 instead of 0.87 ms at the benchmark's sizes)."""
    b = 1
    while b < n:
        if b >= 2 and b + b // 2 >= n:
            return b + b // 2
        b *= 2
    return b


class ModelRunner:
    """Owns the model's parts, the cache and the step's device buffers; `step` is the only way
    tokens go through the model (generation, the scheduler's loop and trace replay all use it)."""

    def __init__(self, config, tensors_or_dir, engine: EngineConfig, arch=None):
        _require_cuda(engine.device)
        from ..models import BuildContext      # registers the built-in architecture
        self.rt = runtime_module()
        self.engine = engine
        self.config = config
        self.device = engine.device
        self.dtype = engine.dtype
        torch.cuda.set_device(self.device)
        arch = arch or architecture_for(config.to_dict())
        manifest = arch.manifest(config)
        if isinstance(tensors_or_dir, (str, os.PathLike)):
            weights = load_safetensors_weights(str(tensors_or_dir), manifest, device=self.device)
        else:
            weights = weights_from_tensors(tensors_or_dir, manifest)
        kernels.set_pdl(bool(engine.pdl))
        self.spec: ModelSpec = arch.build(config, weights, BuildContext(dtype=self.dtype, device=self.device))
        del weights
        if self.dtype == torch.bfloat16:
            # the library product (many rows) must add its split-K partial sums in float32 too
            torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        # what this model needs is compiled now, side by side (a fresh checkout has nothing built):
        # every part names the kernel libraries it launches
        kernels.preload(self.kernel_modules())
        # As in the reference, the longest sequence is the engine's limit, not config.json's
        # max_position_embeddings (crates/engine/src/backend/cpu/mod.rs:49-54): rotation angles are
        # computed from the position itself, so no table length binds them.
        self.max_model_len = engine.max_model_len
        self.pools = CachePools(self.spec, engine.block_size, engine.max_seqs, self.dtype, self.device,
                                num_pages=engine.num_pages, pool_bytes=engine.kv_pool_bytes)
        self.manager = self.pools.manager
        self.max_pages = -(-self.max_model_len // engine.block_size)
        self.rows_cap = engine.max_batch_tokens
        self.seqs_cap = engine.max_seqs
        self.logits_cap = engine.max_batch_tokens
        self.logit_chunk = min(self.logits_cap, max(engine.max_seqs, 64))
        G = self.pools.num_groups
        self.layout = self.rt.step_layout(self.rows_cap, self.seqs_cap, self.logits_cap, G, self.max_pages)
        # a decode step has one row per request, so never more requests than a step has rows
        self.decode_cap = min(self.seqs_cap, self.rows_cap)
        self.decode_layout = self.rt.step_layout(self.decode_cap, self.decode_cap, self.decode_cap, G, self.max_pages)
        total = max(self.layout["total"], self.decode_layout["total"])
        # a ring of pinned staging buffers: the host may run several steps ahead of the device, and a
        # buffer is written again only after the copy that reads it has been executed
        self._stage = [torch.empty(total, dtype=torch.int32, pin_memory=True) for _ in range(4)]
        self._stage_np = [t.numpy() for t in self._stage]
        self._stage_done = [None] * len(self._stage)
        self._stage_next = 0
        self.step_dev = torch.zeros(total, dtype=torch.int32, device=self.device)
        # Decode steps launched ahead of the host's reads alternate between two buffers (`parity`): the
        # metadata of step n + 1 is then copied to the device on a stream of its own WHILE step n runs,
        # instead of between the two (a copy of 20 KB takes some 10 us from request to arrival).
        # Buffer 0 is also the one every other step uses.
        self._devs = [self.step_dev, torch.zeros(total, dtype=torch.int32, device=self.device)]
        self._dev = self.step_dev               # the buffer the step being launched reads
        self._dev_read = [torch.cuda.Event(), torch.cuda.Event()]    # the last launch that reads buffer p has been executed
        self._dev_read_set = [False, False]
        self._uploaded = torch.cuda.Event()
        self._feed_ready = None                 # the buffer whose token rows hold the last decode step's picks
        self._copy_stream = torch.cuda.Stream(device=self.device)
        # workspace: residual + two pending buffers + the largest block + the head's chunk
        self._foldable = None
        if not 0 <= TUNING.few_rows <= kernels.FUSED_GEMM_MAX_ROWS:
            raise ValueError(f"TUNING.few_rows must be 0..{kernels.FUSED_GEMM_MAX_ROWS} (what the fused kernels take), got {TUNING.few_rows}")
        V = self.spec.vocab_size
        self.workspace_bytes = self.workspace_formula(self.rows_cap)
        self.workspace = Workspace(self.workspace_bytes, self.device)
        # scratch of the token pick: a (value, index) pair per row and slice of the vocabulary, or per
        # row and 128-logit tile when the head's own epilogue does the first pass
        pairs = max(kernels.pick_splits(V), kernels.pick_tiles(V))
        self.pick_val = torch.empty(self.logit_chunk * pairs, dtype=torch.float32, device=self.device)
        self.pick_idx = torch.empty(self.logit_chunk * pairs, dtype=torch.int32, device=self.device)
        self.nan_flags = torch.zeros(self.logits_cap, dtype=torch.int32, device=self.device)
        self.sampled = torch.zeros(self.logits_cap, dtype=torch.int32, device=self.device)
        # two pinned buffers: a step's picks may still be unread when the next step writes its own.
        # The pick kernel of a decode step writes them there itself (page-locked host memory that the
        # device can address), so no copy follows the step's last kernel.
        try:
            self._sampled_host_ints = kernels.HostInts((2, self.seqs_cap))
            self.sampled_host = self._sampled_host_ints.tensor
        except KernelError:                     # a device that cannot address host memory: a copy behind every step
            self._sampled_host_ints = None
            self.sampled_host = torch.zeros((2, self.seqs_cap), dtype=torch.int32, pin_memory=True)
        self.sampled_host_np = self.sampled_host.numpy()
        self.steps_run = 0
        self.last_upload_bytes = 0
        self.graphs_enabled = bool(engine.cuda_graphs)
        self.decode_graphs = self.graphs_enabled         # turned off by a decode step that cannot be recorded
        self._graphs = {}
        self._step_graphs = collections.OrderedDict()    # shape class -> (graph, launches); least recently replayed first
        self._step_seen = {}
        self.step_graph_after = int(getattr(engine, "step_graphs", 0))
        self.step_graph_replays = 0
        self._folded = None
        self._graph_launches = {}
        self._graph_pool = None

    # ------------------------------------------------------------------ sizes
    def kernel_modules(self) -> tuple:
        """The kernel libraries this model's parts launch, in first-use order, each once."""
        spec, mods = self.spec, ["sampling"]
        for part in [spec.embedding, *spec.blocks, spec.final_norm, spec.lm_head]:
            mods += list(getattr(part, "kernel_modules", lambda d, r: ())(self.dtype, self.engine.max_batch_tokens))
        return tuple(dict.fromkeys(mods))

    def workspace_formula(self, rows: int) -> int:
        """Peak bytes of the workspace over all steps of at most `rows` tokens, to the byte, read
        off the scopes of `_forward` and `_head` (the reference's arena formula,
        crates/engine/src/model.rs:68-90, for this arrangement; its test that the high-water mark
        of a largest step equals the formula, :400-419, holds here too): the float32 residual,
        two buffers for block outputs still to be added, and the larger of the largest block and
        the head's chunk (logits and the normed rows)."""
        es = 2 if self.dtype == torch.bfloat16 else 4
        h, V = self.spec.hidden_size, self.spec.vocab_size
        resid = aligned(rows * h * 4)
        pending = 2 * aligned(rows * h * es)
        block = max((b.workspace_bytes(rows, h, es) for b in self.spec.blocks), default=0)
        n = min(self.logit_chunk, rows)
        head = aligned(n * V * 4) + self.spec.final_norm.workspace_bytes(n, es)
        total = resid + pending + max(block, head)
        if self._can_fold(1):
            # steps of few rows run in folded form (FoldedState): residual, the next norm's input, the
            # partial sums of squares, and the blocks' folded scratch or the head
            r = min(rows, TUNING.few_rows)
            state = aligned(r * h * 4) + aligned(r * h * 2) + aligned(-(-h // 128) * TUNING.few_rows * 4)
            fblock = max((b.folded_workspace_bytes(r) for b in self.spec.blocks), default=0)
            fhead = aligned(min(self.logit_chunk, r) * V * 4) + self.spec.final_norm.workspace_bytes(min(self.logit_chunk, r), es)
            total = max(total, state + max(fblock, fhead))
        return total

    @classmethod
    def from_dir(cls, model_dir: str, engine: EngineConfig, random_weights_seed: Optional[int] = None,
                 random_weights_std: float = 0.02) -> "ModelRunner":
        """A model folder: config.json and its safetensors. With `random_weights_seed` only
        config.json is read and the weights are drawn on the device from that seed (values as
        `weights.random_tensors` makes them there; a folder written by `write_random_model` is
        drawn on the host and differs)."""
        from .. import models  # noqa: F401  (registers architectures)
        d = read_config_json(model_dir)
        arch = architecture_for(d, os.path.join(model_dir, "config.json"))
        config = arch.config_cls.from_dict(d, os.path.join(model_dir, "config.json"))
        if random_weights_seed is None:
            return cls(config, model_dir, engine, arch)
        _require_cuda(engine.device)
        from ..weights import random_tensors
        tensors = random_tensors(arch.manifest(config), int(random_weights_seed), random_weights_std, engine.dtype, engine.device)
        return cls(config, tensors, engine, arch)

    # ------------------------------------------------------------------ the step
    def context(self, rows: int, seqs: int, arrays=None, layout=None) -> StepContext:
        L, d = layout or self.layout, self._dev
        mp = self.max_pages
        seqs_cap = L["seqs_cap"]

        def vec(key, n):
            o = L[key]
            return d[o:o + n]
        G = self.pools.num_groups
        return StepContext(
            rows=rows, seqs=seqs, dtype=self.dtype,
            tokens=vec("tokens", rows), positions=vec("positions", rows), row_seq=vec("row_seq", rows),
            seq_starts=vec("seq_starts", seqs + 1), context_lens=vec("context_lens", seqs),
            seq_lens=vec("seq_lens", seqs), state_slots=vec("state_slots", seqs),
            logit_rows=vec("logit_rows", L["logits_cap"]),
            slot_mapping=[d[L["slot_mapping"][g]:L["slot_mapping"][g] + rows] for g in range(G)],
            block_tables=[d[L["block_tables"][g]:L["block_tables"][g] + seqs_cap * mp].view(seqs_cap, mp)
                          for g in range(G)],
            workspace=self.workspace,
            max_new=arrays.max_new if arrays is not None else 0,
            max_seq_len=arrays.max_seq_len if arrays is not None else 0, host=arrays,
            decode_only=bool(arrays is not None and arrays.max_new == 1 and arrays.rows == arrays.seqs),
            long_context=bool(arrays is not None and arrays.max_seq_len > TUNING.long_context_keys),
            lead_single=int(arrays.lead_single) if arrays is not None else 0)

    def upload(self, arrays, parity: int = 0, beside: bool = False, first: int = 0) -> None:
        """One pinned host buffer, one asynchronous copy: the step's only host-to-device traffic.
        `beside`: the copy goes to buffer `parity` on the copy stream, ordered only behind the last
        launch that read that buffer, so it runs beside whatever the main stream still has to do; the
        main stream then waits for it. `first`: where the copy starts (a step whose tokens are already
        on the device leaves the token rows, which lie in front, alone)."""
        n = arrays.used
        self.last_upload_bytes = 4 * (n - first)
        i = self._stage_next
        self._stage_next = (i + 1) % len(self._stage)
        if self._stage_done[i] is not None:
            self._stage_done[i].synchronize()        # the copy that last read this buffer has run
        else:
            self._stage_done[i] = torch.cuda.Event()
        arrays.copy_into(self._stage_np[i])
        dst = self._devs[parity]
        if not beside:
            dst[first:n].copy_(self._stage[i][first:n], non_blocking=True)
            self._stage_done[i].record()
            return
        cs = self._copy_stream
        if self._dev_read_set[parity]:
            cs.wait_event(self._dev_read[parity])
        with torch.cuda.stream(cs):
            dst[first:n].copy_(self._stage[i][first:n], non_blocking=True)
            self._stage_done[i].record(cs)
            self._uploaded.record(cs)
        torch.cuda.current_stream().wait_event(self._uploaded)

    def _mark_read(self, parity: int) -> None:
        """Everything launched so far that reads metadata buffer `parity` lies before this point of the stream."""
        self._dev_read[parity].record()
        self._dev_read_set[parity] = True

    def build_arrays(self, entries):
        """Lay out a batch given as runtime StepEntry objects (pages must be reserved already)."""
        return self.rt.build_step(self.manager, entries, self.rows_cap, self.seqs_cap, self.logits_cap,
                                  self.max_pages, self.spec.vocab_size)

    def _can_fold(self, rows: int) -> bool:
        """Few rows and parts that all offer the folded form (see parts.base.FoldedState)."""
        if self._foldable is None:
            spec = self.spec
            from ..parts.rmsnorm import RMSNorm
            self._foldable = bool(
                self.dtype == torch.bfloat16 and self.engine.fold_norms and spec.schedule
                and hasattr(spec.embedding, "forward_folded") and isinstance(spec.final_norm, RMSNorm)
                and all(getattr(spec.blocks[c.layer], "can_fold", lambda: False)() and c.cache is not None and c.write
                        for c in spec.schedule))
        return self._foldable and rows <= TUNING.few_rows

    def _forward_folded(self, ctx: StepContext):
        spec = self.spec
        calls = spec.schedule
        st = spec.embedding.forward_folded(ctx, spec.blocks[calls[0].layer].norm1)
        for i, call in enumerate(calls):
            nxt = spec.blocks[calls[i + 1].layer].norm1 if i + 1 < len(calls) else spec.final_norm
            spec.blocks[call.layer].forward_folded(st, ctx, self.pools.layer_cache(call.cache, call.write), nxt)
        return st

    def _forward(self, ctx: StepContext) -> torch.Tensor:
        """Embedding and every scheduled block; returns (residual, pending): the float32 residual
        and the last block's output that is still to be added to it."""
        spec, ws = self.spec, ctx.workspace
        self._folded = None
        if self._can_fold(ctx.rows):
            self._folded = self._forward_folded(ctx)
            return self._folded.resid, None
        resid = spec.embedding.forward(ctx)
        es_shape = (ctx.rows, spec.hidden_size)
        pend = [ctx.alloc(es_shape), ctx.alloc(es_shape)]
        pending = None
        for i, call in enumerate(spec.schedule):
            block = spec.blocks[call.layer]
            cache = self.pools.layer_cache(call.cache, call.write)
            state = self.pools.state.get(i)
            pending = block.forward(resid, pending, ctx, cache, state, pend[i & 1])
        return resid, pending

    def _head(self, resid, pending, ctx: StepContext, num_logit_rows: int, logits_out: Optional[torch.Tensor],
              layout=None, also=()) -> None:
        """Final norm and output head on the wanted rows, in chunks; a token is picked from every
        row; logits are copied out only where the caller gave a place for them. `also`: functions
        (first row, rows) -> a further place the picked tokens of those rows are written to."""
        spec, L = self.spec, layout or self.layout
        d = self._dev
        V = spec.vocab_size
        if (self.engine.pick_in_head and logits_out is None and self._folded is not None and ctx.decode_only
                and num_logit_rows == ctx.rows <= self.logit_chunk
                and getattr(spec.lm_head, "can_fold", lambda: False)() and hasattr(spec.lm_head, "pick_folded")):
            # every row is wanted, in order, and only its token: the head reads the folded residual and
            # picks in its own epilogue; the logits never exist in memory
            n = num_logit_rows
            tiles = kernels.pick_tiles(V)
            spec.lm_head.pick_folded(self._folded, spec.final_norm.eps, n, d[L["temperature"]:L["temperature"] + n].view(torch.float32),
                                     d[L["seeds"]:L["seeds"] + 2 * n], d[L["sample_steps"]:L["sample_steps"] + n],
                                     self.pick_val[:n * tiles].view(n, tiles), self.pick_idx[:n * tiles].view(n, tiles),
                                     self.nan_flags[:n], self.sampled[:n], [f(0, n) for f in also])
            return
        for c0 in range(0, num_logit_rows, self.logit_chunk):
            n = min(self.logit_chunk, num_logit_rows - c0)
            with ctx.workspace.scope():
                rows = d[L["logit_rows"] + c0:L["logit_rows"] + c0 + n]
                logits = ctx.workspace.alloc((n, V), torch.float32)
                if (self._folded is not None and ctx.decode_only and n == num_logit_rows == ctx.rows
                        and getattr(spec.lm_head, "can_fold", lambda: False)()):
                    # every row is wanted, in order: the head reads the folded residual directly
                    spec.lm_head.forward_folded(self._folded, spec.final_norm.eps, n, logits)
                else:
                    normed = spec.final_norm.forward(resid, pending, ctx, rows=rows, num_rows=n)
                    spec.lm_head.forward(normed, logits)
                temp = d[L["temperature"] + c0:L["temperature"] + c0 + n].view(torch.float32)
                seeds = d[L["seeds"] + 2 * c0:L["seeds"] + 2 * (c0 + n)]
                steps = d[L["sample_steps"] + c0:L["sample_steps"] + c0 + n]
                kernels.pick_tokens(logits, self.sampled[c0:c0 + n], self.nan_flags[c0:c0 + n], self.pick_val,
                                    self.pick_idx, temp, seeds, steps, [f(c0, n) for f in also])
                if logits_out is not None:
                    logits_out[c0:c0 + n].copy_(logits, non_blocking=logits_out.is_cuda)

    def step(self, arrays, logits_out: Optional[torch.Tensor] = None) -> StepResult:
        """Run one batch. `arrays` comes from `build_arrays` or the scheduler. `logits_out`
        (float32 [>=R, vocab], on the device or the host) receives the logits of the wanted rows.
        A picked token of -1 marks a row whose logits held a NaN."""
        T, S, R = arrays.rows, arrays.seqs, arrays.logit_count
        if arrays.max_seq_len > self.max_model_len:
            raise CapacityError("sequence length", int(arrays.max_seq_len), self.max_model_len)
        if logits_out is not None and (logits_out.dim() != 2 or logits_out.shape[0] < R
                                       or logits_out.shape[1] != self.spec.vocab_size or logits_out.dtype != torch.float32):
            raise ShapeError("step", f"logits_out must be float32 [>={R}, {self.spec.vocab_size}]")
        self.upload(arrays)
        self._feed_ready = None
        shape = self._step_shape(arrays) if logits_out is None else None
        if shape is not None:
            entry = self._step_graphs.get(shape)
            if entry is not None:
                self._step_graphs.move_to_end(shape)
                entry[0].replay()
                kernels.count_launches(entry[1])
                self.steps_run += 1
                self.step_graph_replays += 1
                self._mark_read(0)
                return StepResult(self.sampled, None, R)
        self.workspace.reset()
        if shape is None:
            ctx = self.context(T, S, arrays)
        else:
            # a step of a class that may be recorded runs with the class's padded row count and
            # rounded-up longest portion from its first sighting on: launched one by one or
            # replayed, it runs the same kernels (which of them a part picks depends on the rows)
            ctx = self.context(shape[0], S, arrays)
            ctx.max_new = shape[3]
        resid, pending = self._forward(ctx)
        if R:
            self._head(resid, pending, ctx, R, logits_out)
        self.steps_run += 1
        self._mark_read(0)
        if shape is not None:
            if len(self._step_seen) > 4096:
                self._step_seen.clear()                 # a count per shape class ever seen: keep it bounded
            seen = self._step_seen.get(shape, 0) + 1
            self._step_seen[shape] = seen
            if seen >= self.step_graph_after:
                try:
                    self._record_step(shape)
                except Exception as e:      # a part that cannot be recorded (it reads device data on the host, say)
                    self.step_graph_after = 0
                    self._step_graphs.clear()
                    print(f"[vllm_oxide_b200] steps are not recorded as CUDA graphs from here on: {type(e).__name__}: {e}",
                          file=sys.stderr, flush=True)
        return StepResult(self.sampled, logits_out, R)

    # ------------------------------------------------------------------ other steps as CUDA graphs
    STEP_GRAPHS_KEPT = 256

    def _step_shape(self, arrays):
        """The shape class of a step that is no decode step: everything its launches depend on
        besides what lies in the step's device buffers. Rows are rounded up (the rows added are
        padding: position -1, they attend to nothing and write nothing, as in a decode step's
        graph) and so is the longest portion (kernels take it as an upper bound). None: this step
        is not replayed (graphs off, a decode step, no logits wanted)."""
        if not (self.graphs_enabled and self.step_graph_after > 0):
            return None
        return step_shape_class(arrays.rows, arrays.seqs, arrays.logit_count, arrays.max_new, arrays.lead_single,
                                arrays.max_seq_len, self.rows_cap)

    def _record_step(self, shape) -> None:
        """Record the launches of a step of this shape class (nothing runs while recording: the
        step that asked for it has run already)."""
        rows, S, R, longest, lead, long_context = shape
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        n0 = kernels.launch_count()
        with torch.cuda.graph(g, pool=self._graph_pool):
            self.workspace.reset()
            ctx = self.context(rows, S, None)
            ctx.max_new, ctx.lead_single, ctx.long_context = longest, lead, long_context
            resid, pending = self._forward(ctx)
            self._head(resid, pending, ctx, R, None)
        launches = kernels.launch_count() - n0
        kernels.count_launches(-launches)           # recorded, not run
        self._graph_pool = self._graph_pool or g.pool()
        self._step_graphs[shape] = (g, launches)
        while len(self._step_graphs) > self.STEP_GRAPHS_KEPT:
            self._step_graphs.popitem(last=False)   # the one replayed longest ago

    # ------------------------------------------------------------------ decode steps as CUDA graphs
    def _bucket(self, n: int) -> int:
        return min(decode_bucket(n), self.decode_cap)

    def decode_step_graph(self, scheduler, plan, feed_from_device: bool = False, read: bool = True, parity: int = 0,
                          arrays=None):
        """A step in which every request brings exactly one token. Its kernels are the same as any
        step's, but their launches are replayed from a CUDA graph captured once per batch-size
        class (1, 2, 4, ... requests, the batch padded with rows that attend to nothing) and per
        kind of context (long or not: parts may pick other kernels for long contexts), because
        at small batches launching ~10 kernels per layer costs more than running them
        (the reference's estimate: docs/decisions/0003-backend-trait-and-memory.md:51).
        The picked tokens land in pinned host buffer `parity`. With `read` the call waits and
        returns them; without, it returns an event to hand to `read_decode` later. `arrays`: the
        plan's arrays if the caller has built them already (`decode_arrays`)."""
        S = plan.num_entries
        L = self.decode_layout
        if arrays is None:
            arrays = self.decode_arrays(scheduler, plan)
        if arrays.max_seq_len > self.max_model_len:
            raise CapacityError("sequence length", int(arrays.max_seq_len), self.max_model_len)
        if feed_from_device:
            # The tokens of this step are the previous step's picks, taken on the device (the host runs
            # ahead without reading them back; request order must not have changed): a decode step
            # leaves its picks in the token rows of the OTHER buffer itself. The rest of the metadata
            # is copied beside the step in front, which reads its own buffer.
            self.upload(arrays, parity, beside=not read, first=L["positions"])
            if self._feed_ready != parity:
                self._devs[parity][L["tokens"]:L["tokens"] + S].copy_(self.sampled[:S])
        else:
            self.upload(arrays, parity)
        long_context = bool(arrays.max_seq_len > TUNING.long_context_keys)
        if not self.decode_graphs:
            self._decode_eager(S, parity, long_context)      # nothing is recorded: no padding needed
        else:
            b = self._bucket(S)
            key = (b, parity, long_context)
            graph = self._graphs.get(key)
            if graph is None:
                # first step of this class: run it eagerly (that is this step's result), then record
                # the same launches for the steps to come. Padding requests (no rows, state slot 0)
                # are something a recorded step's kernels skip on the device; a model with
                # per-request state is not shown them before it has proved recordable.
                self._decode_eager(S if self.pools.state else b, parity, long_context)
                try:
                    self._record_decode(key)
                except Exception as e:      # a part that cannot be recorded (it reads device data on the host, say)
                    self.decode_graphs = False
                    self._graphs.clear()
                    print(f"[vllm_oxide_b200] decode steps are not recorded as CUDA graphs from here on: {type(e).__name__}: {e}",
                          file=sys.stderr, flush=True)
            else:
                graph.replay()
                kernels.count_launches(self._graph_launches[key])
        self.steps_run += 1
        self._mark_read(parity)
        self._feed_ready = 1 - parity
        if not read:
            ev = torch.cuda.Event()
            ev.record()
            return ev
        # the picked tokens were copied to pinned host memory by the step itself
        torch.cuda.current_stream().synchronize()
        return self.sampled_host_np[parity, :S].tolist()

    def decode_arrays(self, scheduler, plan):
        """The device arrays of a decode step's plan, in the decode steps' layout."""
        L = self.decode_layout
        return scheduler.arrays(plan, L["rows_cap"], L["seqs_cap"], L["logits_cap"], self.max_pages, self.spec.vocab_size)

    def _record_decode(self, key) -> None:
        """Record the launches of a decode step of this class (nothing runs while recording)."""
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        n0 = kernels.launch_count()
        try:
            with torch.cuda.graph(g, pool=self._graph_pool):
                self._decode_eager(*key)
        finally:
            launches = kernels.launch_count() - n0
            kernels.count_launches(-launches)                       # recorded, not run
        self._graph_launches[key] = launches
        self._graphs[key] = g
        self._graph_pool = self._graph_pool or g.pool()

    def read_decode(self, event, count: int, parity: int) -> List[int]:
        """The picked tokens of a decode step launched without reading."""
        event.synchronize()
        return self.sampled_host_np[parity, :count].tolist()

    def _decode_eager(self, b: int, parity: int = 0, long_context: bool = False) -> None:
        L = self.decode_layout
        self.workspace.reset()
        self._dev = self._devs[parity]          # this step's metadata (a recorded step keeps reading this buffer)
        try:
            ctx = self.context(b, b, None, L)
            ctx.decode_only, ctx.max_new, ctx.long_context = True, 1, long_context
            resid, pending = self._forward(ctx)
            # the picks also go to the host buffer of this parity and, as the next decode step's
            # tokens should it be fed from the device, to the token rows of the other metadata buffer:
            # written by the pick kernel itself (two copies behind it cost a replayed step 14 us)
            other, host, t0 = self._devs[1 - parity], self._sampled_host_ints, L["tokens"]
            also = [lambda c0, n: other[t0 + c0:t0 + c0 + n]]
            if host is not None:
                also.append(lambda c0, n: host.at(parity * self.seqs_cap + c0))
            self._head(resid, pending, ctx, b, None, L, also=also)
        finally:
            self._dev = self.step_dev
        if host is None:
            self.sampled_host[parity, :b].copy_(self.sampled[:b], non_blocking=True)

    # ------------------------------------------------------------------ bookkeeping helpers
    def check_kernels(self) -> None:
        """Raise `KernelError` if a bounded wait inside one of the tensor-core kernels expired since
        the last check (their results are then invalid). Reads one word from the device."""
        if self.dtype == torch.bfloat16:
            kernels.gemm_sm100_check()

    def admit(self, request_id: int) -> int:
        """Take a state slot for a request and zero its state. -1 when no slot is free."""
        slot = self.manager.admit(request_id)
        if slot >= 0:
            self.pools.reset_slot(slot)
        return slot

    def step_read_bytes(self, cached_tokens: int) -> int:
        """Bytes a step must read at least: every weight once, plus the cache of `cached_tokens`
        tokens (the contexts of the live requests, summed)."""
        return self.spec.weight_bytes + int(cached_tokens) * self.pools.bytes_per_token()
