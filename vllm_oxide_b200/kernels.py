"""Launch wrappers of the CUDA kernels: every shape, dtype, device and alignment is checked
here, on the host, before a pointer reaches a kernel (the reference's rule for its launch
wrappers, CLAUDE.md:79, and the checks of crates/engine/src/arena/ops.rs:30-268).

There is no CPU path and no fallback: a tensor that is not on a CUDA device, or a kernel
library that cannot be built or loaded, raises.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc.build import load_cuda_module
from .errors import KernelError, ShapeError
from .tuning import TUNING

_CODES = {torch.float32: 0, torch.bfloat16: 1}
_P = ctypes.c_void_p
_I = ctypes.c_int
_L = ctypes.c_longlong
_F = ctypes.c_float

_STATUS = {2001: "bad argument", 2002: "size not supported by this kernel"}


def _code(t: torch.Tensor, op: str) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise ShapeError(op, f"dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _cuda(op: str, *tensors: Optional[torch.Tensor]) -> None:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise KernelError(f"{op}: tensor on {t.device}; the kernels run on a CUDA device only "
                              "(there is no CPU path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ShapeError(op, f"tensors on different devices: {dev} and {t.device}")


def _ptr(t: Optional[torch.Tensor]):
    return _P(t.data_ptr()) if t is not None else _P(0)


def _stream() -> _P:
    # the raw handle straight from the runtime: torch.cuda.current_stream() builds a Python object
    # each time (some 15 us), which adds up over the two hundred launches of a step
    return _P(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


_launches = 0      # kernels of this package launched (or replayed from a graph) so far


def launch_count() -> int:
    return _launches


def count_launches(n: int) -> None:
    """Account for launches that did not pass through a wrapper (a CUDA graph replay)."""
    global _launches
    _launches += n


def _check(status: int, op: str, launches: int = 1) -> None:
    global _launches
    if status != 0:
        what = _STATUS.get(status, f"CUDA error {status}")
        raise KernelError(f"{op}: launch failed: {what}")
    _launches += launches


def _rows_2d(t: torch.Tensor, op: str, name: str) -> None:
    if t.dim() != 2 or t.stride(1) != 1:
        raise ShapeError(op, f"{name} must be 2-D with unit inner stride, got shape {list(t.shape)} "
                             f"strides {list(t.stride())}")


def _int32_vec(t: torch.Tensor, n: int, op: str, name: str) -> None:
    if t.dtype != torch.int32 or t.dim() != 1 or t.numel() < n or not t.is_contiguous():
        raise ShapeError(op, f"{name} must be a contiguous int32 vector of at least {n}, got "
                             f"{t.dtype} {list(t.shape)}")


_fn_cache = {}
_MODULES = ("elementwise", "gemm_f32", "gemm_sm100", "gemm_sm100_pair", "attention", "attention_mma", "attention_sm100", "sampling")

# Per-op device timing, off unless a profile is being taken: CUDA events around each wrapper
# (the reference times ops by wall clock on the CPU and notes that a CUDA backend must use
# events and add no synchronisation, crates/engine/src/arena.rs:66-68,243-255).
_profile = None


class OpProfile:
    """with OpProfile() as p: ...steps...; p.totals() -> [(op, calls, total_ms)] by time."""

    def __init__(self):
        self.events = []

    def __enter__(self):
        global _profile
        _profile = self
        return self

    def __exit__(self, *exc):
        global _profile
        _profile = None
        return False

    def totals(self):
        torch.cuda.synchronize()
        agg = {}
        for name, a, b in self.events:
            c, t = agg.get(name, (0, 0.0))
            agg[name] = (c + 1, t + a.elapsed_time(b))
        return sorted(((n, c, t) for n, (c, t) in agg.items()), key=lambda x: -x[2])


def _timed(fn):
    import functools

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        if _profile is None:
            return fn(*args, **kwargs)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        try:
            return fn(*args, **kwargs)
        finally:
            b.record()
            _profile.events.append((fn.__name__, a, b))
    return wrapper


def _fn(module: str, name: str, argtypes):
    key = (module, name)
    f = _fn_cache.get(key)
    if f is None:
        lib = _load(module)
        try:
            f = getattr(lib, name)
        except AttributeError:
            raise KernelError(f"kernel library '{module}' has no entry point {name}") from None
        f.argtypes = argtypes
        f.restype = _I
        _fn_cache[key] = f
    return f


_pdl_on = False


TENSOR_CORE_HEAD_DIMS = (64, 128)       # head sizes the tensor-core attention kernels are built for


def preload(modules=_MODULES) -> None:
    """Build (side by side) and load kernel modules now, so that compile time is spent at start-up."""
    from .csrc.build import ensure_built
    ensure_built(modules)
    for m in modules:
        _load(m)


def _load(module: str):
    """dlopen a module and hand it the current launch switches."""
    from .csrc.build import _loaded
    fresh = module not in _loaded
    lib = load_cuda_module(module)
    if fresh:
        f = getattr(lib, f"vob_set_pdl_{module}")
        f.argtypes = [_I]
        f.restype = None
        f(1 if _pdl_on else 0)
    return lib


def set_pdl(on: bool) -> None:
    """Switch programmatic dependent launch on or off for every kernel of this package: with it, a
    kernel's set-up (and a matrix product's first weight loads) overlaps the end of the kernel
    before it; each kernel still waits for its predecessors before it reads or writes anything
    they touch. Modules loaded later take the switch over."""
    global _pdl_on
    from .csrc.build import _loaded
    _pdl_on = bool(on)
    for m in _MODULES:
        if m in _loaded:
            f = getattr(_loaded[m], f"vob_set_pdl_{m}")
            f.argtypes = [_I]
            f.restype = None
            f(1 if _pdl_on else 0)


# ------------------------------------------------------------------------------------ embedding
@_timed
def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, err_flag: Optional[torch.Tensor] = None) -> None:
    """out[t] = table[tokens[t]] as float32; `tokens` int32 [T], `out` float32 [T, h]."""
    op = "embed"
    _cuda(op, table, tokens, out, err_flag)
    T = out.shape[0]
    if table.dim() != 2 or not table.is_contiguous():
        raise ShapeError(op, f"table must be contiguous [vocab, h], got {list(table.shape)}")
    _int32_vec(tokens, T, op, "tokens")
    if out.dtype != torch.float32 or out.dim() != 2 or out.shape[1] != table.shape[1] or not out.is_contiguous():
        raise ShapeError(op, f"out must be contiguous float32 [T, {table.shape[1]}], got {out.dtype} {list(out.shape)}")
    f = _fn("elementwise", "vob_embed", [_P, _I, _P, _P, _I, _I, _I, _P, _P])
    _check(f(_ptr(table), _code(table, op), _ptr(tokens), _ptr(out), T, table.shape[1], table.shape[0],
             _ptr(err_flag), _stream()), op)


# ------------------------------------------------------------------------------------ norm
@_timed
def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    """resid (+= delta); out = weight * (x / sqrt(mean(x^2) + eps)). With `rows` (int32 [R]) only
    those rows are normalised into out [R, h] and resid is left as it is."""
    op = "add_rmsnorm"
    _cuda(op, resid, delta, weight, out, rows)
    if resid.dtype != torch.float32 or resid.dim() != 2 or not resid.is_contiguous():
        raise ShapeError(op, f"the residual must be contiguous float32 [T, h], got {resid.dtype} {list(resid.shape)}")
    T, h = resid.shape
    if weight.dtype != torch.float32 or weight.shape != (h,) or not weight.is_contiguous():
        raise ShapeError(op, f"weight must be float32 [{h}], got {weight.dtype} {list(weight.shape)}")
    if delta is not None and (delta.shape != resid.shape or not delta.is_contiguous()):
        raise ShapeError(op, f"delta must be contiguous {list(resid.shape)}, got {list(delta.shape)}")
    R = T
    if rows is not None:
        R = rows.numel()
        _int32_vec(rows, R, op, "rows")
    if out.dim() != 2 or out.shape[0] < R or out.shape[1] != h or not out.is_contiguous():
        raise ShapeError(op, f"out must be contiguous [>={R}, {h}], got {list(out.shape)}")
    if h * 4 > 48 * 1024:
        raise ShapeError(op, f"width {h} is beyond this kernel's limit of {48 * 1024 // 4}")
    f = _fn("elementwise", "vob_add_rmsnorm", [_P, _P, _I, _P, _P, _P, _I, _I, _I, _F, _P])
    _check(f(_ptr(resid), _ptr(delta), _code(delta, op) if delta is not None else 0, _ptr(weight), _ptr(rows),
             _ptr(out), _code(out, op), R, h, float(eps), _stream()), op)


# ------------------------------------------------------------------------------------ rope + cache write
@_timed
def rope_kv_write(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor], positions: torch.Tensor,
                  slots: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor],
                  kcache: Optional[torch.Tensor], vcache: Optional[torch.Tensor],
                  num_heads: int, num_kv_heads: int, head_dim: int) -> None:
    """Rotate q and k in place (float32 angles position * inv_freq) and write k, v to their cache
    slots. q [T, H*hd], k and v [T, KV*hd] may be column slices of one wider tensor. kcache and
    vcache are one layer's pages [num_pages, KV, page_size, hd]."""
    op = "rope_kv_write"
    _cuda(op, q, k, v, positions, slots, inv_freq, kcache, vcache)
    _rows_2d(q, op, "q")
    T = q.shape[0]
    if q.shape[1] != num_heads * head_dim:
        raise ShapeError(op, f"q has {q.shape[1]} columns, expected heads*head_dim = {num_heads * head_dim}")
    if head_dim % 2 != 0:
        raise ShapeError(op, f"head_dim {head_dim} must be even")
    _int32_vec(positions, T, op, "positions")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.shape != (head_dim // 2,) or not inv_freq.is_contiguous()):
        raise ShapeError(op, f"inv_freq must be float32 [{head_dim // 2}], got {inv_freq.dtype} {list(inv_freq.shape)}")
    page_size = 1
    if k is not None:
        _rows_2d(k, op, "k")
        if k.shape != (T, num_kv_heads * head_dim) or k.dtype != q.dtype:
            raise ShapeError(op, f"k must be {q.dtype} [{T}, {num_kv_heads * head_dim}], got {k.dtype} {list(k.shape)}")
        if slots is not None:
            _int32_vec(slots, T, op, "slots")
            if v is None or kcache is None or vcache is None:
                raise ShapeError(op, "a cache write needs v, kcache and vcache")
            _rows_2d(v, op, "v")
            if v.shape != k.shape or v.dtype != q.dtype:
                raise ShapeError(op, f"v must match k, got {v.dtype} {list(v.shape)}")
            for name, c in (("kcache", kcache), ("vcache", vcache)):
                if c.dim() != 4 or c.shape[1] != num_kv_heads or c.shape[3] != head_dim or not c.is_contiguous() or c.dtype != q.dtype:
                    raise ShapeError(op, f"{name} must be contiguous {q.dtype} [pages, {num_kv_heads}, page_size, "
                                         f"{head_dim}], got {c.dtype} {list(c.shape)}")
            if kcache.shape != vcache.shape:
                raise ShapeError(op, "kcache and vcache differ in shape")
            page_size = kcache.shape[2]
    f = _fn("elementwise", "vob_rope_kv_write", [_P, _L, _P, _L, _P, _L, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P])
    _check(f(_ptr(q), q.stride(0), _ptr(k), k.stride(0) if k is not None else 0, _ptr(v),
             v.stride(0) if v is not None else 0, _ptr(positions), _ptr(slots), _ptr(inv_freq), _ptr(kcache),
             _ptr(vcache), _code(q, op), T, num_heads, num_kv_heads if k is not None else 0, head_dim, page_size,
             _stream()), op)


# ------------------------------------------------------------------------------------ swiglu
@_timed
def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, j] = silu(gate_up[t, j]) * gate_up[t, I + j]."""
    op = "swiglu"
    _cuda(op, gate_up, out)
    _rows_2d(gate_up, op, "gate_up")
    T, two_i = gate_up.shape
    if two_i % 2 != 0:
        raise ShapeError(op, f"gate_up has an odd number of columns: {two_i}")
    if out.shape != (T, two_i // 2) or out.dtype != gate_up.dtype or not out.is_contiguous():
        raise ShapeError(op, f"out must be contiguous {gate_up.dtype} [{T}, {two_i // 2}], got {out.dtype} {list(out.shape)}")
    f = _fn("elementwise", "vob_swiglu", [_P, _L, _P, _I, _I, _I, _P])
    _check(f(_ptr(gate_up), gate_up.stride(0), _ptr(out), _code(out, op), T, two_i // 2, _stream()), op)


# ------------------------------------------------------------------------------------ matrix products
@_timed
def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T in true float32 (FMA chains in k order; no tensor cores)."""
    op = "gemm_f32"
    _cuda(op, a, w, out)
    for name, t in (("a", a), ("w", w), ("out", out)):
        _rows_2d(t, op, name)
        if t.dtype != torch.float32:
            raise ShapeError(op, f"{name} must be float32, got {t.dtype}")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise ShapeError(op, f"a has {K} columns, w has {w.shape[1]}")
    if out.shape != (M, N):
        raise ShapeError(op, f"out must be [{M}, {N}], got {list(out.shape)}")
    f = _fn("gemm_f32", "vob_gemm_f32", [_P, _L, _P, _L, _P, _L, _I, _I, _I, _P])
    _check(f(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), M, N, K, _stream()), op)


class _GemmScratch:
    """Per device: the error word that a timed-out wait inside the tensor-core product raises."""

    def __init__(self, device):
        self.err = torch.zeros(1, dtype=torch.int32, device=device)
        self.num_sms = torch.cuda.get_device_properties(device).multi_processor_count


_gemm_scratch = {}


def _scratch_for(device) -> _GemmScratch:
    s = _gemm_scratch.get(device)
    if s is None:
        s = _gemm_scratch[device] = _GemmScratch(device)
    return s


def gemm_sm100_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tcgen05 kernel takes these operands: bfloat16, K a multiple of 8, 16-byte
    aligned rows (what TMA asks for)."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.dim() == 2 and w.dim() == 2
            and a.shape[1] % 8 == 0 and a.stride(1) == 1 and w.stride(1) == 1 and a.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


@_timed
def gemm_sm100(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, splits: Optional[int] = None) -> None:
    """out[T, N] = a[T, K] @ w[N, K]^T on the tcgen05 tensor cores: bfloat16 operands fetched by
    TMA, float32 accumulation in tensor memory, bfloat16 or float32 out. `splits` > 1 (at most 8) splits K over
    the blocks of a cluster (for few tokens); None picks it from the sizes."""
    op = "gemm_sm100"
    _cuda(op, a, w, out)
    if not gemm_sm100_supported(a, w):
        raise ShapeError(op, f"operands must be bfloat16 with K a multiple of 8 and 16-byte aligned rows, got "
                             f"{a.dtype} {list(a.shape)} strides {list(a.stride())} and {w.dtype} {list(w.shape)}")
    T, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (T, N) or out.stride(1) != 1:
        raise ShapeError(op, f"shapes do not fit: a {list(a.shape)}, w {list(w.shape)}, out {list(out.shape)}")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise ShapeError(op, f"out must be bfloat16 or float32, got {out.dtype}")
    sc = _scratch_for(a.device)
    if splits is None:
        f = _fn("gemm_sm100", "vob_gemm_sm100_pick_splits", [_I, _I, _I, _I])
        splits = int(f(T, N, K, sc.num_sms))
    f = _fn("gemm_sm100", "vob_gemm_sm100", [_P, _L, _P, _L, _P, _L, _I, _I, _I, _I, _I, _P, _P])
    _check(f(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), _code(out, op), T, N, K, int(splits),
             _ptr(sc.err), _stream()), op)


@_timed
def gemm_sm100_pair(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[T, N] = a[T, K] @ w[N, K]^T for many rows, on pairs of SMs: tcgen05.mma with cta_group::2
    (256 weight rows x 256 tokens per instruction, operands split over the two blocks' shared
    memory), persistent over output tiles, accumulators double buffered in tensor memory. bfloat16
    operands, bfloat16 or float32 out."""
    op = "gemm_sm100_pair"
    _cuda(op, a, w, out)
    if not gemm_sm100_supported(a, w):
        raise ShapeError(op, f"operands must be bfloat16 with K a multiple of 8 and 16-byte aligned rows, got "
                             f"{a.dtype} {list(a.shape)} strides {list(a.stride())} and {w.dtype} {list(w.shape)}")
    T, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (T, N) or out.stride(1) != 1:
        raise ShapeError(op, f"shapes do not fit: a {list(a.shape)}, w {list(w.shape)}, out {list(out.shape)}")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise ShapeError(op, f"out must be bfloat16 or float32, got {out.dtype}")
    f = _fn("gemm_sm100_pair", "vob_gemm_sm100_pair", [_P, _L, _P, _L, _P, _L, _I, _I, _I, _I, _P, _P])
    _check(f(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), _code(out, op), T, N, K,
             _ptr(_scratch_for(a.device).err), _stream()), op)


@_timed
def gemm_pair_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[T, I] = silu(a @ Wg^T) * (a @ Wu^T) with w_gate_up = [Wg; Wu] ([2I, K], bfloat16) for many rows:
    the two-SM tcgen05 product whose epilogue applies the activation (gate and up never go to memory)."""
    op = "gemm_pair_swiglu"
    _cuda(op, a, w_gate_up, out)
    if not gemm_sm100_supported(a, w_gate_up):
        raise ShapeError(op, "operands must be bfloat16 with K a multiple of 8 and 16-byte aligned rows")
    T, K = a.shape
    if w_gate_up.shape[0] % 2 != 0 or w_gate_up.shape[1] != K:
        raise ShapeError(op, f"w_gate_up must be [2I, {K}], got {list(w_gate_up.shape)}")
    I = w_gate_up.shape[0] // 2
    if out.shape != (T, I) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
        raise ShapeError(op, f"out must be bfloat16 [{T}, {I}], got {out.dtype} {list(out.shape)}")
    f = _fn("gemm_sm100_pair", "vob_gemm_sm100_pair_swiglu", [_P, _L, _P, _L, _P, _L, _I, _I, _I, _P, _P])
    _check(f(_ptr(a), a.stride(0), _ptr(w_gate_up), w_gate_up.stride(0), _ptr(out), out.stride(0), T, I, K,
             _ptr(_scratch_for(a.device).err), _stream()), op)


def _pick_splits(T: int, N: int, K: int, device) -> int:
    f = _fn("gemm_sm100", "vob_gemm_sm100_pick_splits", [_I, _I, _I, _I])
    return int(f(T, N, K, _scratch_for(device).num_sms))


FUSED_GEMM_MAX_ROWS = 64      # what the fused kernels take


@_timed
def gemm_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, splits: Optional[int] = None) -> None:
    """out[T, I] = silu(a @ Wg^T) * (a @ Wu^T) with w_gate_up = [Wg; Wu] ([2I, K], bfloat16): one tcgen05
    kernel with two accumulators whose epilogue applies the activation, for at most 64 rows."""
    op = "gemm_swiglu"
    _cuda(op, a, w_gate_up, out)
    if not gemm_sm100_supported(a, w_gate_up):
        raise ShapeError(op, "operands must be bfloat16 with K a multiple of 8 and 16-byte aligned rows")
    T, K = a.shape
    if w_gate_up.shape[0] % 2 != 0 or w_gate_up.shape[1] != K:
        raise ShapeError(op, f"w_gate_up must be [2I, {K}], got {list(w_gate_up.shape)}")
    I = w_gate_up.shape[0] // 2
    if T > FUSED_GEMM_MAX_ROWS:
        raise ShapeError(op, f"{T} rows: the fused kernel takes at most {FUSED_GEMM_MAX_ROWS}")
    if out.shape != (T, I) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
        raise ShapeError(op, f"out must be bfloat16 [{T}, {I}], got {out.dtype} {list(out.shape)}")
    if splits is None:
        splits = _pick_splits(T, 2 * I, K, a.device)
    f = _fn("gemm_sm100", "vob_gemm_sm100_swiglu", [_P, _L, _P, _L, _P, _L, _I, _I, _I, _I, _P, _P])
    _check(f(_ptr(a), a.stride(0), _ptr(w_gate_up), w_gate_up.stride(0), _ptr(out), out.stride(0), T, I, K, int(splits),
             _ptr(_scratch_for(a.device).err), _stream()), op)


def gemm_qkv_rope_supported(head_dim: int) -> bool:
    return head_dim > 0 and head_dim % 2 == 0 and 128 % head_dim == 0


@_timed
def gemm_qkv_rope(a: torch.Tensor, w_qkv: torch.Tensor, q_out: torch.Tensor, positions: torch.Tensor,
                  slots: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor], kcache: torch.Tensor, vcache: torch.Tensor,
                  num_heads: int, num_kv_heads: int, head_dim: int, splits: Optional[int] = None) -> None:
    """[q | k | v] = a @ [Wq; Wk; Wv]^T in one tcgen05 kernel whose epilogue rotates q and k (float32
    angles position * inv_freq), writes q to q_out [T, H*hd] and the rotated k and v straight to their
    cache slots. At most 64 rows; 128 must be a multiple of head_dim."""
    op = "gemm_qkv_rope"
    _cuda(op, a, w_qkv, q_out, positions, slots, inv_freq, kcache, vcache)
    if not gemm_sm100_supported(a, w_qkv):
        raise ShapeError(op, "operands must be bfloat16 with K a multiple of 8 and 16-byte aligned rows")
    T, K = a.shape
    H, KV, hd = num_heads, num_kv_heads, head_dim
    if not gemm_qkv_rope_supported(hd):
        raise ShapeError(op, f"head_dim {hd}: 128 must be a multiple of it")
    if w_qkv.shape != ((H + 2 * KV) * hd, K):
        raise ShapeError(op, f"w_qkv must be [{(H + 2 * KV) * hd}, {K}], got {list(w_qkv.shape)}")
    if T > FUSED_GEMM_MAX_ROWS:
        raise ShapeError(op, f"{T} rows: the fused kernel takes at most {FUSED_GEMM_MAX_ROWS}")
    if q_out.shape != (T, H * hd) or q_out.dtype != torch.bfloat16 or q_out.stride(1) != 1:
        raise ShapeError(op, f"q_out must be bfloat16 [{T}, {H * hd}], got {q_out.dtype} {list(q_out.shape)}")
    _int32_vec(positions, T, op, "positions")
    if slots is not None:
        _int32_vec(slots, T, op, "slots")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.shape != (hd // 2,) or not inv_freq.is_contiguous()):
        raise ShapeError(op, f"inv_freq must be float32 [{hd // 2}]")
    for name, c in (("kcache", kcache), ("vcache", vcache)):
        if c.dim() != 4 or c.shape[1] != KV or c.shape[3] != hd or not c.is_contiguous() or c.dtype != torch.bfloat16:
            raise ShapeError(op, f"{name} must be contiguous bfloat16 [pages, {KV}, page_size, {hd}], got {c.dtype} {list(c.shape)}")
    if kcache.shape != vcache.shape:
        raise ShapeError(op, "kcache and vcache differ in shape")
    if splits is None:
        splits = _pick_splits(T, (H + 2 * KV) * hd, K, a.device)
    f = _fn("gemm_sm100", "vob_gemm_sm100_qkv",
            [_P, _L, _P, _L, _P, _L, _I, _I, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P])
    _check(f(_ptr(a), a.stride(0), _ptr(w_qkv), w_qkv.stride(0), _ptr(q_out), q_out.stride(0), T, K, int(splits),
             _ptr(_scratch_for(a.device).err), _ptr(positions), _ptr(slots), _ptr(inv_freq), _ptr(kcache), _ptr(vcache),
             H, KV, hd, kcache.shape[2], _stream()), op)


# ------------------------------------------------------------------------------------ folded norms (few rows)
EPI_STORE, EPI_SWIGLU, EPI_QKV, EPI_RESID, EPI_PICK = 0, 1, 2, 3, 4


class _EpiArgs(ctypes.Structure):
    """Mirror of `EpiArgs` in csrc/gemm_sm100.cu."""
    _fields_ = [("positions", _P), ("slots", _P), ("inv_freq", _P), ("kcache", _P), ("vcache", _P),
                ("ssq_in", _P), ("resid", _P), ("next_w", _P), ("xn_out", _P), ("ssq_out", _P),
                ("ld_resid", _L), ("ld_xn", _L),
                ("q_dim", _I), ("kv_dim", _I), ("hd", _I), ("KV", _I), ("page_size", _I),
                ("ssq_tiles", _I), ("ld_ssq", _I), ("inv_h", _F), ("eps", _F), ("pad_", _I),
                ("temperature", _P), ("seeds", _P), ("steps", _P), ("part_val", _P), ("part_idx", _P), ("nan_flags", _P),
                ("ld_part", _L)]


def _dp(t: Optional[torch.Tensor]) -> int:
    return t.data_ptr() if t is not None else 0


@_timed
def embed_fold(table: torch.Tensor, tokens: torch.Tensor, resid: torch.Tensor, next_w: torch.Tensor, xn: torch.Tensor,
               ssq: torch.Tensor, err_flag: Optional[torch.Tensor] = None) -> None:
    """resid[t] = table[tokens[t]] (float32), xn[t] = bf16(resid * next_w), ssq[tile, t] = sum of squares of
    resid over features 128*tile .. +127: the embedding with the first norm's input prepared."""
    op = "embed_fold"
    _cuda(op, table, tokens, resid, next_w, xn, ssq, err_flag)
    T, h = resid.shape
    if table.dim() != 2 or table.shape[1] != h or not table.is_contiguous():
        raise ShapeError(op, f"table must be contiguous [vocab, {h}], got {list(table.shape)}")
    _int32_vec(tokens, T, op, "tokens")
    if resid.dtype != torch.float32 or not resid.is_contiguous() or xn.dtype != torch.bfloat16 or xn.shape != resid.shape or not xn.is_contiguous():
        raise ShapeError(op, "resid must be contiguous float32 [T, h] and xn contiguous bfloat16 of the same shape")
    if next_w.dtype != torch.float32 or next_w.shape != (h,) or not next_w.is_contiguous():
        raise ShapeError(op, f"next_w must be float32 [{h}]")
    tiles = -(-h // 128)
    if ssq.dtype != torch.float32 or ssq.dim() != 2 or ssq.shape[0] < tiles or ssq.shape[1] < T or not ssq.is_contiguous():
        raise ShapeError(op, f"ssq must be contiguous float32 [>={tiles}, >={T}], got {list(ssq.shape)}")
    f = _fn("elementwise", "vob_embed_fold", [_P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _P])
    _check(f(_ptr(table), _code(table, op), _ptr(tokens), _ptr(resid), _ptr(next_w), _ptr(xn), _ptr(ssq), ssq.shape[1], T, h,
             table.shape[0], _ptr(err_flag), _stream()), op)


@_timed
def gemm_fused(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor], mode: int, n_features: int, *,
               ssq_in: Optional[torch.Tensor] = None, eps: float = 0.0, qkv=None, resid=None, pick=None,
               splits: Optional[int] = None) -> None:
    """The tcgen05 product for at most 64 rows with a fused epilogue and, optionally, the RMSNorm of
    its input folded in: `a` holds bf16(x * norm weight), `ssq_in` [tiles, ld] the per-tile sums of
    squares of x, and each token's accumulator is multiplied by 1 / sqrt(mean(x^2) + eps).
      EPI_STORE  out[T, n] (bfloat16 or float32) = result
      EPI_SWIGLU out[T, n] = silu(gate) * up, w = [Wg; Wu] of shape [2n, K]
      EPI_QKV    qkv = (positions, slots, inv_freq, kcache, vcache, H, KV, hd): out[T, H*hd] = rotated q,
                 rotated k and v go to their cache slots
      EPI_RESID  resid = (resid float32 [T, n] updated in place, next_w float32 [n], xn_out bfloat16 [T, n],
                 ssq_out float32 [tiles(n), ld]); out is None
      EPI_PICK   the output head when only the picked tokens are wanted: pick = (temperature float32 [T] or None,
                 seeds int32 [T, 2], steps int32 [T], part_val float32 [T, ld], part_idx int32 [T, ld],
                 nan_flags int32 [T]), ld >= pick_tiles(n): every block leaves the best (value, index) pair of
                 its 128 logits per token (the rule of `pick_tokens`); `pick_final` finishes; out is None"""
    op = "gemm_fused"
    _cuda(op, a, w, out, ssq_in)
    if not gemm_sm100_supported(a, w):
        raise ShapeError(op, "operands must be bfloat16 with K a multiple of 8 and 16-byte aligned rows")
    T, K = a.shape
    if T > FUSED_GEMM_MAX_ROWS:
        raise ShapeError(op, f"{T} rows: the fused kernel takes at most {FUSED_GEMM_MAX_ROWS}")
    w_rows = 2 * n_features if mode == EPI_SWIGLU else n_features
    if w.shape != (w_rows, K):
        raise ShapeError(op, f"w must be [{w_rows}, {K}], got {list(w.shape)}")
    ea = _EpiArgs()
    if ssq_in is not None:
        if ssq_in.dtype != torch.float32 or ssq_in.dim() != 2 or ssq_in.shape[0] != -(-K // 128) or ssq_in.shape[1] < T or not ssq_in.is_contiguous():
            raise ShapeError(op, f"ssq_in must be contiguous float32 [{-(-K // 128)}, >={T}], got {list(ssq_in.shape)}")
        ea.ssq_in, ea.ssq_tiles, ea.ld_ssq, ea.inv_h, ea.eps = _dp(ssq_in), ssq_in.shape[0], ssq_in.shape[1], 1.0 / K, float(eps)
    out_code, ldc, out_ptr = 1, n_features, 0
    if mode in (EPI_STORE, EPI_SWIGLU):
        if out is None or out.shape != (T, n_features) or out.stride(1) != 1 or out.dtype not in (torch.bfloat16, torch.float32):
            raise ShapeError(op, f"out must be [{T}, {n_features}] bfloat16 or float32")
        if mode == EPI_SWIGLU and out.dtype != torch.bfloat16:
            raise ShapeError(op, "the SwiGLU epilogue writes bfloat16")
        out_code, ldc, out_ptr = _code(out, op), out.stride(0), out.data_ptr()
    elif mode == EPI_QKV:
        positions, slots, inv_freq, kcache, vcache, H, KV, hd = qkv
        _cuda(op, positions, slots, inv_freq, kcache, vcache)
        if not gemm_qkv_rope_supported(hd) or n_features != (H + 2 * KV) * hd:
            raise ShapeError(op, f"qkv sizes do not fit: heads {H}/{KV}, head_dim {hd}, features {n_features}")
        if out is None or out.shape != (T, H * hd) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
            raise ShapeError(op, f"out must be bfloat16 [{T}, {H * hd}]")
        _int32_vec(positions, T, op, "positions")
        if slots is not None:
            _int32_vec(slots, T, op, "slots")
        for name, c in (("kcache", kcache), ("vcache", vcache)):
            if c.dim() != 4 or c.shape[1] != KV or c.shape[3] != hd or not c.is_contiguous() or c.dtype != torch.bfloat16:
                raise ShapeError(op, f"{name} must be contiguous bfloat16 [pages, {KV}, page_size, {hd}]")
        if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.shape != (hd // 2,)):
            raise ShapeError(op, f"inv_freq must be float32 [{hd // 2}]")
        ea.positions, ea.slots, ea.inv_freq, ea.kcache, ea.vcache = _dp(positions), _dp(slots), _dp(inv_freq), _dp(kcache), _dp(vcache)
        ea.q_dim, ea.kv_dim, ea.hd, ea.KV, ea.page_size = H * hd, KV * hd, hd, KV, kcache.shape[2]
        ldc, out_ptr = out.stride(0), out.data_ptr()
    elif mode == EPI_RESID:
        r, next_w, xn_out, ssq_out = resid
        _cuda(op, r, next_w, xn_out, ssq_out)
        tiles = -(-n_features // 128)
        if r.dtype != torch.float32 or r.shape != (T, n_features) or r.stride(1) != 1:
            raise ShapeError(op, f"resid must be float32 [{T}, {n_features}]")
        if xn_out.dtype != torch.bfloat16 or xn_out.shape != (T, n_features) or xn_out.stride(1) != 1:
            raise ShapeError(op, f"xn_out must be bfloat16 [{T}, {n_features}]")
        if next_w.dtype != torch.float32 or next_w.shape != (n_features,) or not next_w.is_contiguous():
            raise ShapeError(op, f"next_w must be float32 [{n_features}]")
        if ssq_out.dtype != torch.float32 or ssq_out.dim() != 2 or ssq_out.shape[0] < tiles or ssq_out.shape[1] < T or not ssq_out.is_contiguous():
            raise ShapeError(op, f"ssq_out must be contiguous float32 [>={tiles}, >={T}]")
        ea.resid, ea.next_w, ea.xn_out, ea.ssq_out = _dp(r), _dp(next_w), _dp(xn_out), _dp(ssq_out)
        ea.ld_resid, ea.ld_xn = r.stride(0), xn_out.stride(0)
        if ea.ld_ssq == 0:
            ea.ld_ssq = ssq_out.shape[1]
        elif ea.ld_ssq != ssq_out.shape[1]:
            raise ShapeError(op, "ssq_in and ssq_out must have the same row length")
    elif mode == EPI_PICK:
        temperature, seeds, steps, part_val, part_idx, nan_flags = pick
        _cuda(op, temperature, seeds, steps, part_val, part_idx, nan_flags)
        tiles = pick_tiles(n_features)
        for name, t_, dt in (("part_val", part_val, torch.float32), ("part_idx", part_idx, torch.int32)):
            if t_.dtype != dt or t_.dim() != 2 or t_.shape[0] < T or t_.shape[1] < tiles or not t_.is_contiguous():
                raise ShapeError(op, f"{name} must be contiguous {dt} [>={T}, >={tiles}], got {t_.dtype} {list(t_.shape)}")
        if part_val.shape[1] != part_idx.shape[1]:
            raise ShapeError(op, "part_val and part_idx must have the same row length")
        _int32_vec(nan_flags, T, op, "nan_flags")
        if temperature is not None:
            if temperature.dtype != torch.float32 or temperature.numel() < T or not temperature.is_contiguous():
                raise ShapeError(op, f"temperature must be float32 [{T}]")
            if seeds is None or steps is None or seeds.dtype != torch.int32 or seeds.numel() < 2 * T or not seeds.is_contiguous():
                raise ShapeError(op, f"temperature sampling needs seeds int32 [{T}, 2] and steps")
            _int32_vec(steps, T, op, "steps")
        ea.temperature, ea.seeds, ea.steps = _dp(temperature), _dp(seeds), _dp(steps)
        ea.part_val, ea.part_idx, ea.nan_flags, ea.ld_part = _dp(part_val), _dp(part_idx), _dp(nan_flags), part_val.shape[1]
        out_code = 0
        splits = 1
    else:
        raise ShapeError(op, f"unknown epilogue mode {mode}")
    if splits is None:
        splits = _pick_splits(T, w_rows, K, a.device)
    f = _fn("gemm_sm100", "vob_gemm_sm100_ex", [_P, _L, _P, _L, _P, _L, _I, _I, _I, _I, _I, _I, ctypes.POINTER(_EpiArgs), _P, _P])
    _check(f(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _P(out_ptr), ldc, out_code, T, n_features, K, int(splits), int(mode),
             ctypes.byref(ea), _ptr(_scratch_for(a.device).err), _stream()), op)


def gemm_sm100_test_hooks(extra_tx_bytes: int = 0, wait_limit_ms: float = 0.0) -> None:
    """For the test of the kernels' give-up path only: the next one-block launches of the few-token
    product expect `extra_tx_bytes` more than their loads bring (their waits then run out), and
    waits give up after `wait_limit_ms` (0: the default of two seconds). (0, 0) restores both."""
    f = _fn("gemm_sm100", "vob_gemm_sm100_test_hooks", [_I, ctypes.c_ulonglong])
    _check(f(int(extra_tx_bytes), int(wait_limit_ms * 1e6)), "gemm_sm100_test_hooks", launches=0)


def gemm_sm100_check() -> None:
    """Raise if a bounded wait inside a tcgen05 kernel (matrix product or attention) ever expired
    (reads one word from the device)."""
    for dev, sc in _gemm_scratch.items():
        code = int(sc.err.item())
        if code:
            sc.err.zero_()
            raise KernelError(f"a bounded wait expired inside a tensor-core kernel (code {code}: 1-4 = matrix product: TMA "
                              "producer, MMA issuer, epilogue, peers of a split; 11-21 = attention: 11-12 TMA producer, 13-17 MMA issuer, "
                              "18-21 softmax rows); its result is not valid")


def linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out = a @ w^T. float32 operands: the true 32-bit kernel. bfloat16 operands: this package's
    tcgen05 kernel (TMA operands, float32 accumulation in tensor memory); for many rows, or
    operands TMA cannot address (K not a multiple of 8, unaligned rows), the library product
    (cuBLAS through torch, float32 accumulation; above `TUNING.few_rows` rows), as the reference plans for its own matrix
    products (CLAUDE.md:107). `out` may be bfloat16 or float32."""
    op = "linear"
    if a.dtype == torch.float32:
        gemm_f32(a, w, out)
        return
    _cuda(op, a, w, out)
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise ShapeError(op, f"operands must both be float32 or both bfloat16, got {a.dtype} and {w.dtype}")
    if a.dim() != 2 or w.dim() != 2 or a.shape[1] != w.shape[1] or out.shape != (a.shape[0], w.shape[0]):
        raise ShapeError(op, f"shapes do not fit: a {list(a.shape)}, w {list(w.shape)}, out {list(out.shape)}")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise ShapeError(op, f"out must be bfloat16 or float32, got {out.dtype}")
    if a.shape[0] <= TUNING.few_rows and gemm_sm100_supported(a, w):
        gemm_sm100(a, w, out)
    else:
        _library_gemm_bf16(a, w, out)


@_timed
def _library_gemm_bf16(a, w, out):
    if out.dtype == torch.bfloat16:
        torch.mm(a, w.t(), out=out)
    else:
        torch.mm(a, w.t(), out_dtype=torch.float32, out=out)


# ------------------------------------------------------------------------------------ attention
@_timed
def paged_attention(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                    block_tables: torch.Tensor, row_seq: torch.Tensor, positions: torch.Tensor,
                    num_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: int = 0) -> None:
    """Causal GQA attention of every row of q [T, H*hd] over its request's pages.
    block_tables int32 [S, max_pages]; row_seq, positions int32 [T]; window 0 = all keys."""
    op = "paged_attention"
    _cuda(op, q, out, kcache, vcache, block_tables, row_seq, positions)
    _rows_2d(q, op, "q")
    _rows_2d(out, op, "out")
    T = q.shape[0]
    if q.shape[1] != num_heads * head_dim or out.shape != q.shape or out.dtype != q.dtype:
        raise ShapeError(op, f"q and out must be [{T}, {num_heads * head_dim}] of one dtype, got {list(q.shape)} "
                             f"{q.dtype} and {list(out.shape)} {out.dtype}")
    if num_kv_heads <= 0 or num_heads % num_kv_heads != 0:
        raise ShapeError(op, f"{num_heads} heads are not a multiple of {num_kv_heads} kv heads")
    if head_dim % 8 != 0 or head_dim > 256:
        raise ShapeError(op, f"head_dim {head_dim} is not supported (multiples of 8 up to 256)")
    for name, c in (("kcache", kcache), ("vcache", vcache)):
        if c.dim() != 4 or c.shape[1] != num_kv_heads or c.shape[3] != head_dim or not c.is_contiguous() or c.dtype != q.dtype:
            raise ShapeError(op, f"{name} must be contiguous {q.dtype} [pages, {num_kv_heads}, page_size, {head_dim}], "
                                 f"got {c.dtype} {list(c.shape)}")
    if kcache.shape != vcache.shape:
        raise ShapeError(op, "kcache and vcache differ in shape")
    if kcache.numel() // head_dim >= 2 ** 31:
        raise ShapeError(op, "one layer's cache has 2^31 rows or more")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or not block_tables.is_contiguous():
        raise ShapeError(op, f"block_tables must be contiguous int32 [S, max_pages], got {block_tables.dtype} {list(block_tables.shape)}")
    _int32_vec(row_seq, T, op, "row_seq")
    _int32_vec(positions, T, op, "positions")
    f = _fn("attention", "vob_paged_attention",
            [_P, _L, _P, _L, _P, _P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P])
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache), _code(q, op),
             _ptr(block_tables), block_tables.shape[1], _ptr(row_seq), _ptr(positions), T, num_heads,
             num_kv_heads, head_dim, kcache.shape[2], int(window), float(scale), _stream()), op)


def attn_mma_supported(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, decode: bool) -> bool:
    """Whether the tensor-core attention kernels take these sizes (bfloat16 only)."""
    if head_dim not in TENSOR_CORE_HEAD_DIMS:
        return False                      # answered here: a model of another head size never builds the module
    f = _fn("attention_mma", "vob_attn_mma_supported", [_I, _I, _I, _I, _I])
    return bool(f(num_heads, num_kv_heads, head_dim, page_size, int(decode)))


def _attn_common_checks(op, q, out, kcache, vcache, block_tables, num_heads, num_kv_heads, head_dim):
    _cuda(op, q, out, kcache, vcache, block_tables)
    _rows_2d(q, op, "q")
    _rows_2d(out, op, "out")
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16 or vcache.dtype != torch.bfloat16:
        raise ShapeError(op, "the tensor-core attention kernels are bfloat16 only")
    if q.shape[1] != num_heads * head_dim or out.shape != q.shape:
        raise ShapeError(op, f"q and out must be [T, {num_heads * head_dim}], got {list(q.shape)} and {list(out.shape)}")
    for name, c in (("kcache", kcache), ("vcache", vcache)):
        if c.dim() != 4 or c.shape[1] != num_kv_heads or c.shape[3] != head_dim or not c.is_contiguous():
            raise ShapeError(op, f"{name} must be contiguous [pages, {num_kv_heads}, page_size, {head_dim}], got {list(c.shape)}")
    if kcache.shape != vcache.shape:
        raise ShapeError(op, "kcache and vcache differ in shape")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or not block_tables.is_contiguous():
        raise ShapeError(op, "block_tables must be contiguous int32 [S, max_pages]")
    if q.stride(0) % 8 != 0 or q.data_ptr() % 16 != 0 or out.stride(0) % 2 != 0 or out.data_ptr() % 4 != 0:
        raise ShapeError(op, "q rows must be 16-byte aligned and out rows 4-byte aligned")
    if not attn_mma_supported(num_heads, num_kv_heads, head_dim, kcache.shape[2], False):
        raise ShapeError(op, f"sizes not supported by the tensor-core kernels: heads {num_heads}/{num_kv_heads}, "
                             f"head_dim {head_dim}, page {kcache.shape[2]} (head_dim 64 or 128, page size dividing 64)")


@_timed
def attn_prefill_mma(q, out, kcache, vcache, block_tables, seq_starts, context_lens, num_seqs: int, max_new: int,
                     num_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: int = 0) -> None:
    """Tensor-core attention for portions of prompts and mixed batches (bfloat16). q/out [T, H*hd];
    seq_starts int32 [S+1] (first row of each request), context_lens int32 [S] (keys cached before
    the step), max_new = the longest portion."""
    op = "attn_prefill_mma"
    if not scale > 0:
        raise ShapeError(op, f"the score scale must be positive, got {scale}")
    _attn_common_checks(op, q, out, kcache, vcache, block_tables, num_heads, num_kv_heads, head_dim)
    _cuda(op, seq_starts, context_lens)
    _int32_vec(seq_starts, num_seqs + 1, op, "seq_starts")
    _int32_vec(context_lens, num_seqs, op, "context_lens")
    if block_tables.shape[0] < num_seqs:
        raise ShapeError(op, f"block_tables has {block_tables.shape[0]} rows for {num_seqs} requests")
    f = _fn("attention_mma", "vob_attn_prefill_mma",
            [_P, _L, _P, _L, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _P])
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache), _ptr(block_tables),
             block_tables.shape[1], _ptr(seq_starts), _ptr(context_lens), num_seqs, max_new, num_heads, num_kv_heads,
             head_dim, kcache.shape[2], int(window), float(scale), _stream()), op)


def attn_prefill_sm100_supported(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, max_pages: int) -> bool:
    """Whether the tcgen05 attention kernel for prompt portions takes these sizes (bfloat16, no window)."""
    if head_dim not in TENSOR_CORE_HEAD_DIMS:
        return False
    f = _fn("attention_sm100", "vob_attn_prefill_sm100_supported", [_I, _I, _I, _I, _I])
    return bool(f(num_heads, num_kv_heads, head_dim, page_size, max_pages))


@_timed
def attn_prefill_sm100(q, out, kcache, vcache, block_tables, seq_starts, context_lens, num_seqs: int, max_new: int,
                       num_heads: int, num_kv_heads: int, head_dim: int, scale: float) -> None:
    """Attention for portions of prompts and mixed batches on the tcgen05 tensor cores (bfloat16,
    head_dim 64 or 128, no window): Q, K and V tiles by TMA straight from the pages of the cache, scores
    and output in tensor memory. Arguments as `attn_prefill_mma`."""
    op = "attn_prefill_sm100"
    if not scale > 0:
        raise ShapeError(op, f"the score scale must be positive, got {scale}")
    _cuda(op, q, out, kcache, vcache, block_tables, seq_starts, context_lens)
    _rows_2d(q, op, "q")
    _rows_2d(out, op, "out")
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16 or vcache.dtype != torch.bfloat16:
        raise ShapeError(op, "the tensor-core attention kernels are bfloat16 only")
    if q.shape[1] != num_heads * head_dim or out.shape != q.shape:
        raise ShapeError(op, f"q and out must be [T, {num_heads * head_dim}], got {list(q.shape)} and {list(out.shape)}")
    for name, c in (("kcache", kcache), ("vcache", vcache)):
        if c.dim() != 4 or c.shape[1] != num_kv_heads or c.shape[3] != head_dim or not c.is_contiguous():
            raise ShapeError(op, f"{name} must be contiguous [pages, {num_kv_heads}, page_size, {head_dim}], got {list(c.shape)}")
    if kcache.shape != vcache.shape:
        raise ShapeError(op, "kcache and vcache differ in shape")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or not block_tables.is_contiguous():
        raise ShapeError(op, "block_tables must be contiguous int32 [S, max_pages]")
    if block_tables.shape[0] < num_seqs:
        raise ShapeError(op, f"block_tables has {block_tables.shape[0]} rows for {num_seqs} requests")
    for name, t in (("q", q), ("out", out)):
        if t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0:
            raise ShapeError(op, f"{name} rows must be 16-byte aligned")
    if not attn_prefill_sm100_supported(num_heads, num_kv_heads, head_dim, kcache.shape[2], block_tables.shape[1]):
        raise ShapeError(op, f"sizes not supported: heads {num_heads}/{num_kv_heads}, head_dim {head_dim}, page "
                             f"{kcache.shape[2]}, {block_tables.shape[1]} pages per request (head_dim 64 or 128, at most 128 "
                             "heads per kv head, page size a power of two from 8 to 128)")
    _int32_vec(seq_starts, num_seqs + 1, op, "seq_starts")
    _int32_vec(context_lens, num_seqs, op, "context_lens")
    f = _fn("attention_sm100", "vob_attn_prefill_sm100",
            [_P, _L, _L, _P, _L, _P, _P, _L, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P, _P])
    _check(f(_ptr(q), q.shape[0], q.stride(0), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache), kcache.shape[0],
             _ptr(block_tables), block_tables.shape[1], _ptr(seq_starts), _ptr(context_lens), num_seqs, max_new, num_heads,
             num_kv_heads, head_dim, kcache.shape[2], float(scale), _ptr(_scratch_for(q.device).err), _stream()), op)


@_timed
def attn_decode_mma(q, out, kcache, vcache, block_tables, positions, num_heads: int, num_kv_heads: int, head_dim: int,
                    scale: float, window: int = 0, splits: int = 1, partials=None, arrived=None) -> None:
    """Tensor-core attention for a step of single tokens, row i belonging to request i (bfloat16).
    With splits > 1 (at most 8) each request's keys are shared out over the blocks of a cluster,
    which merge their partial results through distributed shared memory. With `partials` (float32,
    `attn_decode_partial_floats` elements) and `arrived` (int32 zeros, one per request and kv head;
    the kernel leaves them zero) up to 64 blocks share a request without a cluster and merge
    through global memory: for few requests with long contexts."""
    op = "attn_decode_mma"
    if not scale > 0:
        raise ShapeError(op, f"the score scale must be positive, got {scale}")
    _attn_common_checks(op, q, out, kcache, vcache, block_tables, num_heads, num_kv_heads, head_dim)
    _cuda(op, positions)
    S = q.shape[0]
    _int32_vec(positions, S, op, "positions")
    if block_tables.shape[0] < S:
        raise ShapeError(op, f"block_tables has {block_tables.shape[0]} rows for {S} requests")
    if num_heads // num_kv_heads > 16:
        raise ShapeError(op, f"{num_heads // num_kv_heads} heads per kv head: the decode kernel takes at most 16")
    if (partials is None) != (arrived is None):
        raise ShapeError(op, "partials and arrived go together")
    most = 8 if partials is None else 64
    if not 1 <= splits <= most:
        raise ShapeError(op, f"splits must be 1..{most}, got {splits}")
    if partials is not None:
        _cuda(op, partials, arrived)
        need = attn_decode_partial_floats(S, num_kv_heads, head_dim, splits)
        if partials.dtype != torch.float32 or not partials.is_contiguous() or partials.numel() < need or partials.data_ptr() % 16:
            raise ShapeError(op, f"partials must be contiguous float32, 16-byte aligned, with at least {need} elements")
        if arrived.dtype != torch.int32 or not arrived.is_contiguous() or arrived.numel() < S * num_kv_heads:
            raise ShapeError(op, f"arrived must be contiguous int32 with at least {S * num_kv_heads} elements")
    f = _fn("attention_mma", "vob_attn_decode_mma",
            [_P, _L, _P, _L, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P, _P, _P])
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache), _ptr(block_tables),
             block_tables.shape[1], _ptr(positions), S, num_heads, num_kv_heads, head_dim, kcache.shape[2], int(window),
             float(scale), int(splits), _ptr(partials), _ptr(arrived), _stream()), op)


def attn_decode_partial_floats(num_seqs: int, num_kv_heads: int, head_dim: int, splits: int) -> int:
    """Elements of the float32 scratch that `attn_decode_mma` needs for its merge through global memory."""
    return num_seqs * num_kv_heads * splits * (16 * head_dim + 32)


# ------------------------------------------------------------------------------------ sampling
def pick_tiles(vocab: int) -> int:
    """Pairs per row that the output head's picking epilogue (EPI_PICK) leaves: one per 128 logits."""
    return -(-int(vocab) // 128)


class HostInts:
    """A page-locked host buffer of int32 that kernels write to directly (`also` of the pick
    functions): `tensor` is the host's view, `address` what the device reaches it under."""

    def __init__(self, shape):
        self.tensor = torch.zeros(shape, dtype=torch.int32, pin_memory=True)
        f = _fn("sampling", "vob_host_device_pointer", [_P, _P])
        dev = ctypes.c_void_p()
        rc = f(_P(self.tensor.data_ptr()), ctypes.byref(dev))
        if rc != 0 or not dev.value:
            raise KernelError(f"the device cannot address page-locked host memory (error {rc})")
        self.address = int(dev.value)

    def at(self, element: int) -> "_Address":
        if not 0 <= element <= self.tensor.numel():
            raise ShapeError("HostInts", f"element {element} lies outside {self.tensor.numel()} elements")
        return _Address(self.address + 4 * element, self.tensor.numel() - element)


class _Address:
    """A raw device-reachable address with the int32 elements that follow it."""

    def __init__(self, address: int, elements: int):
        self.address, self.elements = address, elements


def _also_pointers(op: str, also, rows: int):
    """Up to two further places the picked tokens go to: int32 device tensors or addresses of a `HostInts`."""
    if len(also) > 2:
        raise ShapeError(op, f"at most two further destinations, got {len(also)}")
    ptrs = []
    for a in also:
        if isinstance(a, _Address):
            if a.elements < rows:
                raise ShapeError(op, f"a further destination has room for {a.elements} of {rows} tokens")
            ptrs.append(_P(a.address))
        else:
            _cuda(op, a)
            _int32_vec(a, rows, op, "a further destination")
            ptrs.append(_ptr(a))
    return ptrs + [_P(0)] * (2 - len(ptrs))


@_timed
def pick_final(part_val: torch.Tensor, part_idx: torch.Tensor, rows: int, vocab: int, nan_flags: torch.Tensor,
               out: torch.Tensor, also=()) -> None:
    """The pick's second pass alone: out[r] = index of the best of row r's (value, index) pairs
    (part_val / part_idx [>= rows, pairs per row]); -1 for a row whose NaN flag is up (the flag is cleared).
    `also`: up to two further places the same tokens are written to."""
    op = "pick_final"
    _cuda(op, part_val, part_idx, nan_flags, out)
    if (part_val.dtype != torch.float32 or part_idx.dtype != torch.int32 or part_val.dim() != 2 or part_val.shape != part_idx.shape
            or part_val.shape[0] < rows or not part_val.is_contiguous() or not part_idx.is_contiguous()):
        raise ShapeError(op, f"part_val float32 and part_idx int32 must be contiguous [>={rows}, pairs], got {list(part_val.shape)} "
                             f"and {list(part_idx.shape)}")
    _int32_vec(out, rows, op, "out")
    _int32_vec(nan_flags, rows, op, "nan_flags")
    a, b = _also_pointers(op, also, rows)
    f = _fn("sampling", "vob_pick_final_to", [_P, _P, _I, _I, _I, _P, _P, _P, _P, _P])
    _check(f(_ptr(part_val), _ptr(part_idx), rows, part_val.shape[1], int(vocab), _ptr(nan_flags), _ptr(out), a, b, _stream()), op)


def pick_splits(vocab: int) -> int:
    f = _fn("sampling", "vob_pick_splits", [_I])
    return int(f(vocab))


@_timed
def pick_tokens(logits: torch.Tensor, out: torch.Tensor, nan_flags: torch.Tensor, scratch_val: torch.Tensor,
                scratch_idx: torch.Tensor, temperature: Optional[torch.Tensor] = None,
                seeds: Optional[torch.Tensor] = None, steps: Optional[torch.Tensor] = None, also=()) -> None:
    """One token per row of float32 logits [R, V]: greedy where temperature is 0 or absent,
    Gumbel-max sampling elsewhere. seeds int32 [R, 2] (low, high word), steps int32 [R]
    (index of the generated token), nan_flags int32 [R] raised for rows that hold a NaN.
    scratch_val float32 and scratch_idx int32 need R * pick_splits(V) elements each.
    `also`: up to two further places the same tokens are written to."""
    op = "pick_tokens"
    _cuda(op, logits, out, nan_flags, scratch_val, scratch_idx, temperature, seeds, steps)
    _rows_2d(logits, op, "logits")
    if logits.dtype != torch.float32:
        raise ShapeError(op, f"logits must be float32, got {logits.dtype}")
    R, V = logits.shape
    splits = pick_splits(V)
    _int32_vec(out, R, op, "out")
    _int32_vec(nan_flags, R, op, "nan_flags")
    if scratch_val.dtype != torch.float32 or scratch_val.numel() < R * splits or not scratch_val.is_contiguous():
        raise ShapeError(op, f"scratch_val must hold {R * splits} float32")
    if scratch_idx.dtype != torch.int32 or scratch_idx.numel() < R * splits or not scratch_idx.is_contiguous():
        raise ShapeError(op, f"scratch_idx must hold {R * splits} int32")
    if temperature is not None:
        if temperature.dtype != torch.float32 or temperature.numel() < R or not temperature.is_contiguous():
            raise ShapeError(op, f"temperature must be float32 [{R}]")
        if seeds is None or steps is None:
            raise ShapeError(op, "temperature sampling needs seeds and steps")
        if seeds.dtype != torch.int32 or seeds.numel() < 2 * R or not seeds.is_contiguous():
            raise ShapeError(op, f"seeds must be int32 [{R}, 2]")
        _int32_vec(steps, R, op, "steps")
    a, b = _also_pointers(op, also, R)
    f = _fn("sampling", "vob_pick_tokens_to", [_P, _L, _I, _I, _P, _P, _P, _I, _P, _P, _P, _P, _P, _P, _P])
    _check(f(_ptr(logits), logits.stride(0), R, V, _ptr(temperature), _ptr(seeds), _ptr(steps), splits,
             _ptr(scratch_val), _ptr(scratch_idx), _ptr(nan_flags), _ptr(out), a, b, _stream()), op, launches=2)
