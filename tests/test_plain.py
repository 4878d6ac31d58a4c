"""The plain implementation checks itself against facts the reference's tests state (no GPU)."""
import math

import pytest
import torch

from tests.plain import llama_plain as plain
from tests.test_config import LLAMA_1B
from tests.util import TINY_A, TINY_B, make_model_dir, random_tokens


def test_llama3_bands():
    # crates/engine/src/backend/cpu/rope.rs:108-128
    inv = plain.rope_inv_freq(LLAMA_1B)
    raw = [500000.0 ** (-(2 * i) / 64) for i in range(32)]
    assert inv.shape == (32,) and float(inv[0]) == 1.0
    assert abs(float(inv[31]) - raw[31] / 32) < 1e-9
    assert all(float(inv[i]) > float(inv[i + 1]) for i in range(31))
    assert all(raw[i] / 32 * (1 - 1e-6) <= float(inv[i]) <= raw[i] * (1 + 1e-6) for i in range(32))
    plain_inv = plain.rope_inv_freq({**LLAMA_1B, "rope_scaling": None})
    assert all(abs(float(plain_inv[i]) - raw[i]) < 1e-7 for i in range(32))


def test_rope_position_zero_is_identity_and_norm_is_kept():
    # crates/engine/src/backend/cpu/rope.rs:131-161
    cfg = TINY_B.to_dict()
    inv = plain.rope_inv_freq(cfg)
    x = torch.randn(2, 3 * 32, dtype=torch.float64)
    y = plain.rope(x, [0, 37], inv, 32)
    assert torch.equal(y[0], x[0])
    assert abs(float(y[1].norm() - x[1].norm())) < 1e-12
    th = 37.0 * float(inv[5])
    a, b = float(x[1, 5]), float(x[1, 16 + 5])
    assert abs(float(y[1, 5]) - (a * math.cos(th) - b * math.sin(th))) < 1e-6
    assert abs(float(y[1, 21]) - (b * math.cos(th) + a * math.sin(th))) < 1e-6


def test_rms_norm_and_swiglu_values():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    out = plain.rms_norm(x, torch.tensor([2.0, 0.5], dtype=torch.float64), 0.0)
    r = math.sqrt(12.5)
    assert torch.allclose(out, torch.tensor([[2 * 3 / r, 0.5 * 4 / r]], dtype=torch.float64))
    g, u = torch.tensor([0.0, 1.0, -2.0], dtype=torch.float64), torch.tensor([5.0, 2.0, 3.0], dtype=torch.float64)
    want = [0.0, 1 / (1 + math.exp(-1)) * 2, -2 / (1 + math.exp(2)) * 3]
    assert torch.allclose(plain.swiglu(g, u), torch.tensor(want, dtype=torch.float64))


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    T, H, KV, hd = 9, 4, 2, 8
    q, k, v = (torch.randn(T, n * hd, dtype=torch.float64) for n in (H, KV, KV))
    out = plain.causal_attention(q, k, v, H, KV, hd)
    assert torch.allclose(out[0, :hd], v[0, :hd])                      # the first row sees one key
    k2, v2 = k.clone(), v.clone()
    k2[5:], v2[5:] = 9.0, -9.0                                         # the future must not matter
    assert torch.equal(plain.causal_attention(q, k2, v2, H, KV, hd)[:5], out[:5])
    assert torch.allclose(plain.causal_attention(q * 0, k, v, H, KV, hd)[3, :hd], v[:4, :hd].mean(0))   # uniform weights
    # heads 0,1 read kv head 0; heads 2,3 read kv head 1
    v3 = v.clone()
    v3[:, hd:] += 1.0
    o3 = plain.causal_attention(q, k, v3, H, KV, hd)
    assert torch.allclose(o3[:, :2 * hd], out[:, :2 * hd]) and torch.allclose(o3[:, 2 * hd:], out[:, 2 * hd:] + 1.0)
    w = plain.causal_attention(q, k, v, H, KV, hd, window=3)
    assert torch.allclose(w[:3], out[:3]) and not torch.allclose(w[5], out[5])
    assert torch.allclose(w[8], plain.causal_attention(q[6:], k[6:], v[6:], H, KV, hd)[2])


def test_argmax_cases():
    # crates/engine/src/backend/cpu/tests.rs:129-144
    f = lambda xs: plain.argmax_first(torch.tensor(xs, dtype=torch.float64))
    assert f([1, 5, 5, -1]) == 1 and f([0, 0, 0]) == 0 and f([-3, -2, -2, -9]) == 1
    with pytest.raises(ValueError):
        f([1.0, float("nan")])


def test_temperature_pick_follows_softmax():
    logits = torch.tensor([2.0, 1.0, 0.0, -1.0], dtype=torch.float64)
    counts = [0] * 4
    n = 4000
    for s in range(n):
        counts[plain.temperature_pick(logits, 0.7, seed=1234, step=s)] += 1
    p = torch.softmax(logits / 0.7, 0)
    for i in range(4):
        assert abs(counts[i] / n - float(p[i])) < 4 * math.sqrt(float(p[i]) * (1 - float(p[i])) / n) + 1e-3
    assert plain.temperature_pick(logits, 0.0, 1, 1) == 0
    assert plain.temperature_pick(logits, 0.7, 5, 9) == plain.temperature_pick(logits, 0.7, 5, 9)


def test_forward_shapes_and_prefix_property(tmp_path):
    for name, cfgobj in (("A", TINY_A), ("B", TINY_B)):
        d = make_model_dir(tmp_path, name)
        cfg, tensors = plain.load_model(d)
        toks = random_tokens(12, cfgobj.vocab_size, 3)
        full = plain.forward(cfg, tensors, toks)
        assert full.shape == (12, cfgobj.vocab_size)
        assert torch.allclose(plain.forward(cfg, tensors, toks[:7]), full[:7], atol=1e-12)     # causal: a prefix is a prefix
        out = plain.greedy_generate(cfg, tensors, toks, 3)
        assert out[0] == plain.argmax_first(full[-1]) and len(out) == 3
        stop = out[1]
        assert plain.greedy_generate(cfg, tensors, toks, 3, stop=stop)[-1] == stop
