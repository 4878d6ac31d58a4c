"""Interfaces of the parts a decoder is put together from, and of what a step hands them.

A model is data: a list of blocks, and a list that says in which order they run and which
cache each call uses (`ModelSpec.schedule`). A block arranges a mixer and a feed-forward
around two norms; which mixer, feed-forward, norm and position encoding a block gets is the
architecture builder's choice per layer, taken from the configuration. No part knows which
model it is in: sizes and constants arrive as constructor parameters, per-step facts arrive
in a `StepContext`.

What each kind of part must offer:

* Mixer        - `cache_spec()` (pages it needs: which tensors a page holds, for all keys or a
                 window of them; or None), `state_spec()` (fixed-size per-request state, or None),
                 `forward(x, ctx, cache, state, out=None) -> [T, hidden]` in the compute dtype.
* FeedForward  - `forward(x, ctx, out=None) -> [T, hidden]`.
* Norm         - `forward(resid, delta, ctx, rows=None) -> normed`; adds `delta` into the
                 float32 residual first (the residual sum is kept in 32-bit).
* PositionEncoding - whatever its mixer asks of it; the rotary part offers `inv_freq`.
Every part may also offer `workspace_bytes(rows)` (what it takes from the step's workspace, to
the byte), `kernel_modules(dtype, max_rows)` (the kernel libraries it launches, so that an
engine compiles them at its start) and `weight_bytes()`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch


# ------------------------------------------------------------------------------ cache / state needs
@dataclass(frozen=True)
class PagedTensorSpec:
    """One tensor of a paged cache: per token `heads` vectors of `width` elements, laid out as
    [num_pages, heads, page_size, width] (head-major inside a page). `dtype` None means the
    engine's compute dtype."""
    heads: int
    width: int
    dtype: Optional[torch.dtype] = None


@dataclass(frozen=True)
class CacheSpec:
    """Pages a mixer needs. The mixer says which tensors a page holds: keys and values of
    `num_kv_heads` x `head_dim` (the default, `CacheSpec(kv_heads, head_dim)`), or any other set
    given as `tensors` (one latent vector per token, keys and values of different widths, ...),
    and whether every token is kept ("full") or only the last `window` ("window")."""
    num_kv_heads: int = 0
    head_dim: int = 0
    kind: str = "full"          # "full": every key is kept; "window": the last `window` keys
    window: int = 0
    tensors: Tuple[PagedTensorSpec, ...] = ()

    def paged_tensors(self) -> Tuple[PagedTensorSpec, ...]:
        """The tensors of one page: `tensors` if given, else a key and a value tensor."""
        if self.tensors:
            return self.tensors
        kv = PagedTensorSpec(self.num_kv_heads, self.head_dim)
        return (kv, kv)

    def group_key(self) -> Tuple:
        return (self.kind, self.window, self.paged_tensors())


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size state per request: one tensor of `shape` per state slot, zeroed at admission."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class LayerCache:
    """One cache of one call in the schedule: this layer's pages (one tensor per entry of its
    `CacheSpec.paged_tensors()`, each [num_pages, heads, page_size, width]) and which group's
    block tables address them. `k` and `v` are the first two (the default key / value pair)."""
    tensors: Tuple[torch.Tensor, ...]
    group: int
    write: bool = True          # False: the call reads a cache that another call wrote

    @property
    def k(self) -> torch.Tensor:
        return self.tensors[0]

    @property
    def v(self) -> torch.Tensor:
        return self.tensors[1]

    @property
    def page_size(self) -> int:
        return self.tensors[0].shape[2]


# ------------------------------------------------------------------------------ per-step facts
_ELEMENT_SIZE = {torch.float32: 4, torch.bfloat16: 2, torch.float16: 2, torch.int32: 4, torch.int64: 8, torch.uint8: 1,
                 torch.int8: 1, torch.float64: 8}


def aligned(nbytes: int) -> int:
    """Bytes one workspace allocation of `nbytes` takes (allocations are multiples of 256 bytes)."""
    return (int(nbytes) + 255) & ~255


class Workspace:
    """A bump allocator over one device buffer: a step's activations live here, so that a step
    allocates nothing and its tensors sit at the same addresses every time. The reference's
    per-step arena (crates/engine/src/arena.rs:92-158) with scopes that rewind on close. Every
    allocation takes `aligned(nbytes)` bytes, so a part can say to the byte what it will take."""

    def __init__(self, nbytes: int, device):
        self.buf = torch.empty(max(aligned(nbytes), 256), dtype=torch.uint8, device=device)
        self.top = 0
        self.high_water = 0

    def alloc(self, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * _ELEMENT_SIZE[dtype]
        start = self.top                       # a multiple of 256: every allocation is rounded up
        if start + aligned(nbytes) > self.buf.numel():
            from ..errors import CapacityError
            raise CapacityError("step workspace", start + aligned(nbytes), self.buf.numel())
        self.top = start + aligned(nbytes)
        self.high_water = max(self.high_water, self.top)
        return self.buf[start:start + nbytes].view(dtype).view(*shape)

    def reset(self) -> None:
        self.top = 0

    class _Scope:
        def __init__(self, ws):
            self.ws = ws

        def __enter__(self):
            self.mark = self.ws.top
            return self.ws

        def __exit__(self, *exc):
            self.ws.top = self.mark
            return False

    def scope(self) -> "_Scope":
        return Workspace._Scope(self)


@dataclass
class StepContext:
    """Everything a part may read about the current step. Device tensors are views into the
    step's packed int32 buffer; they hold `rows_cap` / `seqs_cap` entries of which the first
    `rows` / `seqs` are real (the rest is padding that attends to nothing and writes nothing).

    Steps are recorded as CUDA graphs and replayed for later steps of the same shape class, so
    what a part launches may depend only on the host facts below that make up the class (`rows`,
    `seqs`, `max_new` as an upper bound, `decode_only`, `lead_single`, `long_context`) and on its
    own constants; everything else must be read on the device, from the tensors. `max_seq_len`
    and `host` are there for checks and debugging only (a recording is made with neither)."""
    rows: int                       # rows the kernels run over (real rows, or the padded count)
    seqs: int
    dtype: torch.dtype              # compute dtype of activations and cache
    tokens: torch.Tensor            # int32 [rows]
    positions: torch.Tensor         # int32 [rows]   position of each row in its request
    row_seq: torch.Tensor           # int32 [rows]   which request of the batch a row belongs to
    seq_starts: torch.Tensor        # int32 [seqs+1] first row of each request
    context_lens: torch.Tensor      # int32 [seqs]   keys cached before this step
    seq_lens: torch.Tensor          # int32 [seqs]   keys after this step
    state_slots: torch.Tensor       # int32 [seqs]   state slot of each request
    logit_rows: torch.Tensor        # int32 [R]
    slot_mapping: List[torch.Tensor]   # per group: int32 [rows] cache slot of each row (-1: none)
    block_tables: List[torch.Tensor]   # per group: int32 [seqs, max_pages]
    workspace: Workspace
    max_new: int = 0                # longest portion in the batch (host fact)
    max_seq_len: int = 0            # longest context after the step (host fact)
    decode_only: bool = False       # every request brings exactly one token and row i is request i
    lead_single: int = 0            # the first so many requests bring exactly one token each (host fact):
                                    # rows 0 .. lead_single - 1 are theirs, row i belonging to request i
    long_context: bool = False      # some request is longer than TUNING.long_context_keys (host fact; a replayed
                                    # step was recorded with the same value)
    host: Optional[object] = None   # the host-side StepArrays (ids, counts) for parts that want them

    def alloc(self, shape, dtype=None) -> torch.Tensor:
        return self.workspace.alloc(shape, dtype or self.dtype)


@dataclass
class FoldedState:
    """The residual stream of a step of few rows with the next norm's input prepared ("folded"
    form): the kernel that produced `resid` also wrote `xn` = bf16(resid * weight of the norm that
    follows) and `ssq` [tile, row] = sums of squares of `resid` over tiles of 128 features. The
    matrix product that consumes `xn` multiplies its result by 1 / sqrt(mean(resid^2) + eps), so no
    norm kernel runs. Parts that can work on this form offer `can_fold()` and `forward_folded`."""
    resid: torch.Tensor     # float32 [rows, hidden]
    xn: torch.Tensor        # bfloat16 [rows, hidden]
    ssq: torch.Tensor       # float32 [ceil(hidden / 128), TUNING.few_rows]




# ------------------------------------------------------------------------------ part interfaces
class Mixer:
    """Mixes information between the tokens of a request (attention here)."""

    def cache_spec(self) -> Optional[CacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def workspace_bytes(self, rows: int) -> int:
        """Bytes this part takes from the step's workspace in a step of `rows` rows or fewer."""
        return 0

    def kernel_modules(self, dtype: torch.dtype, max_rows: int) -> Tuple[str, ...]:
        """Names of the kernel libraries (csrc/<name>.cu) this part launches in an engine of
        this compute dtype whose steps have at most `max_rows` rows."""
        return ()

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[LayerCache],
                state: Optional[torch.Tensor], out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x [T, hidden] in the compute dtype -> [T, hidden]. `out`, if given, is where the
        result should go (a part may ignore it and return a tensor of its own)."""
        raise NotImplementedError


class FeedForward:
    def workspace_bytes(self, rows: int) -> int:
        return 0

    def kernel_modules(self, dtype: torch.dtype, max_rows: int) -> Tuple[str, ...]:
        return ()

    def forward(self, x: torch.Tensor, ctx: StepContext, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class Norm:
    # True for a norm that is a per-token scale times a per-feature weight (`weight`, `eps`):
    # that form commutes with a matrix product and can be folded into it (see FoldedState).
    scale_and_weight = False

    def workspace_bytes(self, rows: int, act_bytes: int) -> int:
        return 0

    def kernel_modules(self, dtype: torch.dtype, max_rows: int) -> Tuple[str, ...]:
        return ()

    def forward(self, resid: torch.Tensor, delta: Optional[torch.Tensor], ctx: StepContext,
                rows: Optional[torch.Tensor] = None, num_rows: Optional[int] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding:
    pass


# ------------------------------------------------------------------------------ a model as data
@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order: run `layer` with cache number `cache` (None: the mixer keeps
    no pages). Naming a layer twice runs it twice (with two caches, or sharing one); `write`
    False lets a call read a cache that an earlier call of the same step wrote."""
    layer: int
    cache: Optional[int] = None
    write: bool = True


@dataclass
class ModelSpec:
    embedding: object                   # .forward(ctx) -> float32 residual [rows, hidden]
    blocks: List[object]                # Block parts
    schedule: List[LayerCall]
    final_norm: Norm
    lm_head: object                     # .forward(normed, ctx, out) -> float32 logits
    hidden_size: int
    vocab_size: int
    max_position: Optional[int] = None  # longest position the position encodings allow
    eos_token_ids: Tuple[int, ...] = ()
    weight_bytes: int = 0               # bytes a decode step must read of the weights
