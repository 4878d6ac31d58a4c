"""A plain, slow implementation of the Llama dense decoder: the oracle of every test.

It rests on the reference's formulas, read from its CPU backend (the reference is a Rust
workspace; no Rust toolchain exists on the build machine, so its code could not be compiled
or run here, and no golden outputs of it exist). Each function restates one part and cites
the lines it was read from, by the file's path inside the reference project.

Whole sequences, no cache, no batching, one request at a time, float64 arithmetic on the
CPU (the reference computes in float32; float64 makes this the common target that a
float32 and a bfloat16 engine are both compared with). It shares no code with the product:
it parses config.json with `json`, reads tensors with the third-party `safetensors`
package, and uses torch only as an array library.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch

F64 = torch.float64


# ----------------------------------------------------------------------------- loading
def load_model(model_dir: str):
    """config.json as a dict and every tensor widened to float64 (bf16 -> f32 is exact:
    crates/engine/src/weights.rs:93-95)."""
    from safetensors.torch import load_file
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    tensors = {k: v.to(F64) for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items()}
    return cfg, tensors


def head_dim_of(cfg: dict) -> int:
    # crates/engine/src/config.rs:74-76 (hidden / heads); config.json's own head_dim wins if present
    return int(cfg["head_dim"]) if cfg.get("head_dim") else cfg["hidden_size"] // cfg["num_attention_heads"]


# ----------------------------------------------------------------------------- parts
def embedding(table: torch.Tensor, tokens: List[int]) -> torch.Tensor:
    """out[t] = table[tokens[t]]   (crates/engine/src/backend/cpu/mod.rs:172-180)."""
    return torch.stack([table[int(t)] for t in tokens])


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """w * (x * 1/sqrt(mean(x^2) + eps)), the weight multiplied last
    (crates/engine/src/backend/cpu/mod.rs:182-197)."""
    out = torch.empty_like(x)
    for r in range(x.shape[0]):
        mean_square = float((x[r] * x[r]).sum()) / x.shape[1]
        inv_rms = 1.0 / math.sqrt(mean_square + eps)
        out[r] = weight * (x[r] * inv_rms)
    return out


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """out[t, o] = sum_k x[t, k] * W[o, k]; W is [out, in], no bias
    (crates/engine/src/backend/cpu/mod.rs:199-229)."""
    return x @ weight.t()


def rope_inv_freq(cfg: dict) -> torch.Tensor:
    """Inverse frequencies [head_dim/2] as float32 values, llama3-scaled when config.json has
    rope_scaling (crates/engine/src/backend/cpu/rope.rs:36-61). The reference computes every
    step in float32; so does this, except the power, which is taken in float64 and rounded
    (the reference's f32 powf may differ from it in the last bit)."""
    d = head_dim_of(cfg)
    base = float(cfg.get("rope_theta", 10000.0))
    f32 = torch.float32
    inv = []
    for i in range(d // 2):
        expo = torch.tensor((2 * i), dtype=f32) / torch.tensor(d, dtype=f32)
        p = torch.tensor(math.pow(base, float(expo)), dtype=f32)
        inv.append(torch.tensor(1.0, dtype=f32) / p)
    rs = cfg.get("rope_scaling")
    if rs is None:
        return torch.stack(inv)
    assert rs.get("rope_type", rs.get("type")) == "llama3"
    factor = torch.tensor(rs["factor"], dtype=f32)
    low = torch.tensor(rs["low_freq_factor"], dtype=f32)
    high = torch.tensor(rs["high_freq_factor"], dtype=f32)
    old_ctx = torch.tensor(rs["original_max_position_embeddings"], dtype=f32)
    low_freq_wavelen = old_ctx / low
    high_freq_wavelen = old_ctx / high
    two_pi = torch.tensor(2.0, dtype=f32) * torch.tensor(math.pi, dtype=f32)
    out = []
    for v in inv:
        wavelen = two_pi / v
        if wavelen < high_freq_wavelen:
            out.append(v)                                   # high frequency: untouched
        elif wavelen > low_freq_wavelen:
            out.append(v / factor)                          # low frequency: fully scaled
        else:
            smooth = (old_ctx / wavelen - low) / (high - low)
            out.append((1.0 - smooth) * v / factor + smooth * v)
    return torch.stack(out)


def rope(x: torch.Tensor, positions: List[int], inv_freq: torch.Tensor, head_dim: int) -> torch.Tensor:
    """Rotate-half RoPE on every head of x [T, heads*head_dim]; the angle p*inv_freq is
    formed in float32 (crates/engine/src/backend/cpu/rope.rs:64-99)."""
    half = head_dim // 2
    out = x.clone()
    for t, p in enumerate(positions):
        theta = (torch.tensor(float(p), dtype=torch.float32) * inv_freq).to(F64)   # f32 product
        cos, sin = torch.cos(theta), torch.sin(theta)
        for h0 in range(0, x.shape[1], head_dim):
            x1 = x[t, h0:h0 + half]
            x2 = x[t, h0 + half:h0 + head_dim]
            out[t, h0:h0 + half] = x1 * cos - x2 * sin
            out[t, h0 + half:h0 + head_dim] = x2 * cos + x1 * sin
    return out


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, num_heads: int,
                     num_kv_heads: int, head_dim: int, window: Optional[int] = None,
                     scale: Optional[float] = None) -> torch.Tensor:
    """Two-pass-softmax causal GQA attention of one whole sequence; row t sees keys 0..t
    (crates/engine/src/backend/cpu/attention.rs:76-128). `window` (not a reference feature)
    limits row t to its last `window` keys, t included."""
    T = q.shape[0]
    group = num_heads // num_kv_heads
    scale = 1.0 / math.sqrt(head_dim) if scale is None else scale
    out = torch.zeros_like(q)
    for t in range(T):
        first = 0 if window is None else max(0, t + 1 - window)
        for h in range(num_heads):
            kvh = h // group
            qv = q[t, h * head_dim:(h + 1) * head_dim]
            keys = k[first:t + 1, kvh * head_dim:(kvh + 1) * head_dim]
            vals = v[first:t + 1, kvh * head_dim:(kvh + 1) * head_dim]
            scores = (keys @ qv) * scale
            e = torch.exp(scores - scores.max())
            w = e / e.sum()
            out[t, h * head_dim:(h + 1) * head_dim] = w @ vals
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """gate / (1 + exp(-gate)) * up   (crates/engine/src/backend/cpu/mod.rs:341-349)."""
    return gate / (1.0 + torch.exp(-gate)) * up


def feed_forward(x: torch.Tensor, w_gate, w_up, w_down) -> torch.Tensor:
    """down(silu(gate(x)) * up(x))   (crates/engine/src/model.rs:325-331)."""
    return linear(swiglu(linear(x, w_gate), linear(x, w_up)), w_down)


def attention_block(x, tensors, prefix, cfg, positions, inv_freq):
    """q,k,v projections, RoPE on q and k, causal attention, output projection
    (crates/engine/src/model.rs:302-321)."""
    H, KV, hd = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"], head_dim_of(cfg)
    q = rope(linear(x, tensors[prefix + "self_attn.q_proj.weight"]), positions, inv_freq, hd)
    k = rope(linear(x, tensors[prefix + "self_attn.k_proj.weight"]), positions, inv_freq, hd)
    v = linear(x, tensors[prefix + "self_attn.v_proj.weight"])
    a = causal_attention(q, k, v, H, KV, hd)
    return linear(a, tensors[prefix + "self_attn.o_proj.weight"])


def forward(cfg: dict, tensors: Dict[str, torch.Tensor], tokens: List[int]) -> torch.Tensor:
    """Logits [T, vocab] at every position of one whole sequence
    (crates/engine/src/model.rs:269-356, without its last-row selection)."""
    eps = float(cfg["rms_norm_eps"])
    inv_freq = rope_inv_freq(cfg)
    positions = list(range(len(tokens)))
    x = embedding(tensors["model.embed_tokens.weight"], tokens)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        normed = rms_norm(x, tensors[p + "input_layernorm.weight"], eps)
        x = x + attention_block(normed, tensors, p, cfg, positions, inv_freq)
        normed = rms_norm(x, tensors[p + "post_attention_layernorm.weight"], eps)
        x = x + feed_forward(normed, tensors[p + "mlp.gate_proj.weight"], tensors[p + "mlp.up_proj.weight"],
                             tensors[p + "mlp.down_proj.weight"])
    normed = rms_norm(x, tensors["model.norm.weight"], eps)
    head = tensors["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else tensors["lm_head.weight"]
    return linear(normed, head)


# ----------------------------------------------------------------------------- picking tokens
def argmax_first(row: torch.Tensor) -> int:
    """First index of the maximum; NaN is an error (crates/engine/src/backend/cpu/mod.rs:370-388)."""
    best = 0
    for i in range(row.shape[0]):
        v = float(row[i])
        if math.isnan(v):
            raise ValueError("argmax: NaN in logits")
        if v > float(row[best]):
            best = i
    return best


def _mix32(x: int) -> int:
    """The 32-bit finaliser of the engine's counter-based generator (its own design; the
    reference samples greedily only)."""
    x &= 0xFFFFFFFF
    x ^= x >> 16
    x = (x * 0x7FEB352D) & 0xFFFFFFFF
    x ^= x >> 15
    x = (x * 0x846CA68B) & 0xFFFFFFFF
    x ^= x >> 16
    return x


def gumbel_noise(seed: int, step: int, index: int) -> float:
    """g = -log(-log(u)), u in (0,1) from a hash of (seed, generated index, vocabulary index),
    in float32 steps as the kernel takes them."""
    import numpy as np
    key = _mix32((seed & 0xFFFFFFFF) ^ _mix32(((seed >> 32) + 0x85EBCA6B) & 0xFFFFFFFF))
    ctr = _mix32(key ^ _mix32((step + 0x9E3779B9) & 0xFFFFFFFF))
    h = _mix32(ctr ^ (index & 0xFFFFFFFF))
    u = (np.float32(h >> 8) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)
    return float(-np.log(-np.log(u, dtype=np.float32), dtype=np.float32))


def temperature_pick(row: torch.Tensor, temperature: float, seed: int, step: int) -> int:
    """Gumbel-max: argmax_i(logit_i / temperature + g_i); equal in law to sampling from
    softmax(logits / temperature)."""
    if temperature == 0.0:
        return argmax_first(row)
    import numpy as np
    best, best_v = 0, -math.inf
    for i in range(row.shape[0]):
        v = float(np.float32(np.float32(float(row[i])) / np.float32(temperature)) + np.float32(gumbel_noise(seed, step, i)))
        if v > best_v:
            best, best_v = i, v
    return best


def greedy_generate(cfg, tensors, prompt: List[int], max_new: int, stop: Optional[int] = None) -> List[int]:
    """The reference's driver loop with whole-sequence recomputation instead of a cache:
    the stop token is kept and ends the output (crates/engine/src/generate.rs:104-122)."""
    seq = list(prompt)
    out = []
    for _ in range(max_new):
        tok = argmax_first(forward(cfg, tensors, seq)[-1])
        out.append(tok)
        if stop is not None and tok == stop:
            break
        seq.append(tok)
    return out
