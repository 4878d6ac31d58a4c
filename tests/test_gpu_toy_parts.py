"""Toy parts defined here run through the unchanged framework, chosen layer by layer: a
feed-forward with routing (top-1 of a few experts, router in float32) and a position encoding
that is no rotation (a learned table added to the mixer's input) beside the framework's own
attention and SwiGLU. It is no model of anyone's. Registered as an architecture of its own, built
from a model folder, replayed whole, in portions and mixed, and driven by the scheduler."""
import json
import os

import pytest
import torch

from tests.plain import llama_plain as plain
from tests.util import max_rel_diff

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
NAME = "ToyRoutedAbsolute"


def _register():
    from dataclasses import dataclass
    from vllm_oxide_b200.config import Architecture, register_architecture
    from vllm_oxide_b200.parts import Attention, Block, Embedding, FeedForward, LayerCall, LMHead, Mixer, ModelSpec, RMSNorm, Rotary, SwiGLU
    from vllm_oxide_b200.parts.base import PositionEncoding
    from vllm_oxide_b200.weights import TensorSpec

    @dataclass(frozen=True)
    class ToyConfig:
        hidden: int
        heads: int
        kv_heads: int
        head_dim: int
        inter: int
        experts: int
        expert_inter: int
        vocab: int
        max_pos: int
        eps: float

        @classmethod
        def from_dict(cls, d, where="config.json"):
            return cls(*[d["toy_" + k] for k in ("hidden", "heads", "kv_heads", "head_dim", "inter", "experts", "expert_inter",
                                                 "vocab", "max_pos", "eps")])

        def to_dict(self):
            d = {"toy_" + k: getattr(self, k) for k in ("hidden", "heads", "kv_heads", "head_dim", "inter", "experts",
                                                       "expert_inter", "vocab", "max_pos", "eps")}
            d["architectures"] = [NAME]
            return d

    class LearnedPositions(PositionEncoding):
        """A table [max_pos, hidden]; its mixer adds row `position` to its input."""

        def __init__(self, table, dtype, device):
            self.table = table.to(device=device, dtype=dtype)

    class PositionedAttention(Mixer):
        """The framework's attention (no rotation) behind a position encoding of another kind."""

        def __init__(self, inner, positions):
            self.inner, self.positions = inner, positions

        def cache_spec(self):
            return self.inner.cache_spec()

        def workspace_bytes(self, rows):
            return self.inner.workspace_bytes(rows) + rows * self.positions.table.shape[1] * 4 + 256

        def forward(self, x, ctx, cache, state, out=None):
            pos = ctx.positions[:x.shape[0]].long().clamp_(min=0)
            return self.inner.forward(x + self.positions.table[pos], ctx, cache, state, out)

    class TopOneExperts(FeedForward):
        """out = p_e(x) * expert_e(x), e = the expert with the largest router logit; the router's
        logits and softmax in float32. The experts are the framework's SwiGLU parts."""

        def __init__(self, router, experts, dtype, device):
            self.router = router.to(device=device, dtype=torch.float32)
            self.experts = experts
            self.dtype = dtype

        def workspace_bytes(self, rows):
            return max(e.workspace_bytes(rows) for e in self.experts)

        def forward(self, x, ctx, out=None):
            logits = x.float() @ self.router.t()
            p, e = torch.softmax(logits, dim=-1).max(dim=-1)
            res = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
            for i, expert in enumerate(self.experts):
                rows = (e == i).nonzero().flatten()
                if rows.numel():
                    with ctx.workspace.scope():
                        y = expert.forward(x[rows].contiguous(), ctx)
                        res[rows] = y.float() * p[rows, None]
            return res.to(self.dtype)

    def manifest(c):
        qd, kd = c.heads * c.head_dim, c.kv_heads * c.head_dim
        m = {"emb": TensorSpec((c.vocab, c.hidden)), "final": TensorSpec((c.hidden,), init="ones"),
             "pos": TensorSpec((c.max_pos, c.hidden))}
        for i in range(2):
            m[f"l{i}.n1"] = TensorSpec((c.hidden,), init="ones")
            m[f"l{i}.n2"] = TensorSpec((c.hidden,), init="ones")
            for n, shape in (("q", (qd, c.hidden)), ("k", (kd, c.hidden)), ("v", (kd, c.hidden)), ("o", (c.hidden, qd))):
                m[f"l{i}.{n}"] = TensorSpec(shape)
        for n, shape in (("gate", (c.inter, c.hidden)), ("up", (c.inter, c.hidden)), ("down", (c.hidden, c.inter))):
            m[f"l0.{n}"] = TensorSpec(shape)
        m["l1.router"] = TensorSpec((c.experts, c.hidden))
        for e in range(c.experts):
            for n, shape in (("gate", (c.expert_inter, c.hidden)), ("up", (c.expert_inter, c.hidden)), ("down", (c.hidden, c.expert_inter))):
                m[f"l1.e{e}.{n}"] = TensorSpec(shape)
        return m

    def build(c, w, ctx):
        dt, dev = ctx.dtype, ctx.device
        emb = Embedding(w.take("emb"), dt, dev)

        def attn(i, position):
            return Attention(w.take(f"l{i}.q"), w.take(f"l{i}.k"), w.take(f"l{i}.v"), w.take(f"l{i}.o"), c.heads, c.kv_heads,
                             c.head_dim, position=position, dtype=dt, device=dev)
        # layer 0: rotary attention + dense SwiGLU; layer 1: learned positions + routed experts
        b0 = Block(RMSNorm(w.take("l0.n1"), c.eps, dev), attn(0, Rotary(c.head_dim, 10000.0, None, dev)),
                   RMSNorm(w.take("l0.n2"), c.eps, dev), SwiGLU(w.take("l0.gate"), w.take("l0.up"), w.take("l0.down"), dt, dev))
        experts = [SwiGLU(w.take(f"l1.e{e}.gate"), w.take(f"l1.e{e}.up"), w.take(f"l1.e{e}.down"), dt, dev) for e in range(c.experts)]
        b1 = Block(RMSNorm(w.take("l1.n1"), c.eps, dev), PositionedAttention(attn(1, None), LearnedPositions(w.take("pos"), dt, dev)),
                   RMSNorm(w.take("l1.n2"), c.eps, dev), TopOneExperts(w.take("l1.router"), experts, dt, dev))
        spec = ModelSpec(embedding=emb, blocks=[b0, b1], schedule=[LayerCall(0, 0), LayerCall(1, 1)],
                         final_norm=RMSNorm(w.take("final"), c.eps, dev), lm_head=LMHead(emb.table),
                         hidden_size=c.hidden, vocab_size=c.vocab)
        w.finish()
        return spec

    register_architecture(Architecture(NAME, ToyConfig, manifest, build), replace=True)
    return ToyConfig


def _plain_logits(model_dir, tokens, router_gaps=None):
    """The toy model on one whole sequence in float64, written out directly. `router_gaps`
    collects, per position, the gap between the two largest router probabilities."""
    c = json.load(open(os.path.join(model_dir, "config.json")))
    from safetensors.torch import load_file
    t = {k: v.double() for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items()}
    H, KV, hd, eps = c["toy_heads"], c["toy_kv_heads"], c["toy_head_dim"], c["toy_eps"]
    T = len(tokens)
    positions = list(range(T))
    inv = plain.rope_inv_freq({"head_dim": hd, "hidden_size": H * hd, "num_attention_heads": H, "rope_theta": 10000.0})
    x = plain.embedding(t["emb"], tokens)
    # layer 0
    n = plain.rms_norm(x, t["l0.n1"], eps)
    q = plain.rope(plain.linear(n, t["l0.q"]), positions, inv, hd)
    k = plain.rope(plain.linear(n, t["l0.k"]), positions, inv, hd)
    x = x + plain.linear(plain.causal_attention(q, k, plain.linear(n, t["l0.v"]), H, KV, hd), t["l0.o"])
    x = x + plain.feed_forward(plain.rms_norm(x, t["l0.n2"], eps), t["l0.gate"], t["l0.up"], t["l0.down"])
    # layer 1
    n = plain.rms_norm(x, t["l1.n1"], eps) + t["pos"][:T]
    a = plain.causal_attention(plain.linear(n, t["l1.q"]), plain.linear(n, t["l1.k"]), plain.linear(n, t["l1.v"]), H, KV, hd)
    x = x + plain.linear(a, t["l1.o"])
    n = plain.rms_norm(x, t["l1.n2"], eps)
    probs = torch.softmax(plain.linear(n, t["l1.router"]), dim=-1)
    p, e = probs.max(dim=-1)
    if router_gaps is not None:
        top2 = probs.topk(2, dim=-1).values
        router_gaps.extend((top2[:, 0] - top2[:, 1]).tolist())
    ff = torch.zeros_like(x)
    for r in range(T):
        i = int(e[r])
        ff[r] = p[r] * plain.feed_forward(n[r:r + 1], t[f"l1.e{i}.gate"], t[f"l1.e{i}.up"], t[f"l1.e{i}.down"])[0]
    x = x + ff
    return plain.linear(plain.rms_norm(x, t["final"], eps), t["emb"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_routing_and_positions_run_through_the_unchanged_framework(tmp_path, dtype):
    from vllm_oxide_b200.config import EngineConfig, unregister_architecture
    from vllm_oxide_b200.engine import LLM, ModelRunner
    from vllm_oxide_b200.replay.trace import TraceSession
    from vllm_oxide_b200.sampling import SamplingParams
    from vllm_oxide_b200.weights import write_random_model
    ToyConfig = _register()
    try:
        d = str(tmp_path / "toy")
        write_random_model(d, ToyConfig(48, 3, 1, 16, 80, 3, 64, 61, 96, 1e-5), seed=9, std=0.15, norm_jitter=0.2)
        eng = EngineConfig(max_batch_tokens=96, max_seqs=3, max_model_len=96, block_size=8, num_pages=24, dtype=dtype, cuda_graphs=False)
        runner = ModelRunner.from_dir(d, eng)
        assert runner.pools.num_groups == 1                # both attention layers need the same kind of cache
        s = TraceSession(runner)
        reqs = {"a": [(7 * i + 2) % 61 for i in range(50)], "b": [(5 * i + 11) % 61 for i in range(23)]}
        gaps = {k: [] for k in reqs}
        want = {k: _plain_logits(d, v, gaps[k]) for k, v in reqs.items()}
        f32 = dtype == "float32"
        tol = 2e-5 if f32 else 3e-2

        def check(got, name, first):
            """float32: every position. bfloat16: positions whose routing is no near-tie (a flipped
            expert is a different function, not a rounding; the routed layer is the last one, so a
            flip touches its own position only)."""
            ref = want[name][first:first + got.shape[0]]
            checked = 0
            for i in range(got.shape[0]):
                if not f32 and gaps[name][first + i] < 0.05:
                    continue
                assert max_rel_diff(got[i], ref[i]) <= tol, (name, first + i)
                checked += 1
            return checked

        whole = s.run_step({"step": 0, "entries": [{"id": "a", "tokens": reqs["a"], "want": list(range(50))}], "end": ["a"]})
        assert check(whole, "a", 0) >= 25
        # portions of both requests side by side, down to single tokens; pages are taken again
        cuts = {"a": [9, 1, 24, 2, 14], "b": [2, 16, 1, 3, 1]}
        pos = {"a": 0, "b": 0}
        for i in range(5):
            entries = [{"id": k, "tokens": reqs[k][pos[k]:pos[k] + cuts[k][i]], "want": list(range(cuts[k][i]))} for k in ("a", "b")]
            out = s.run_step({"step": 1 + i, "entries": entries, "end": []})
            check(out[:cuts["a"][i]], "a", pos["a"])
            check(out[cuts["a"][i]:], "b", pos["b"])
            for k in pos:
                pos[k] += cuts[k][i]
        s.run_step({"step": 9, "entries": [], "end": ["a", "b"]})
        assert runner.manager.check_invariants() == "" and runner.manager.num_free_pages(0) == 24
        if f32:
            # greedy generation over the scheduler
            llm = LLM(runner)
            prompts = [reqs["a"][:7], reqs["b"][:12], reqs["a"][5:9]]
            for prompt, o in zip(prompts, llm.generate(prompts, SamplingParams(max_new_tokens=4, stop_token_ids=()))):
                seq = list(prompt)
                for tok in o.token_ids:
                    assert tok == int(_plain_logits(d, seq)[-1].argmax())
                    seq.append(tok)
    finally:
        unregister_architecture(NAME)
