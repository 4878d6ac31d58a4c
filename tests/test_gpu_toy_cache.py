"""A toy mixer whose paged cache is NOT a key / value pair: per token it keeps one latent vector
(compute dtype, width 12) and one float32 gate of another width, as its `CacheSpec.tensors` says.
Defined here, registered as an architecture of its own, built from a model folder and stepped by the
unchanged framework: the pools allocate what the spec names, the cache manager hands out pages, block
tables and slots, replay cuts the work four ways. It is no model of anyone's:
    l_t = x_t W_l,  g_t = sigmoid(x_t w_g),  out_t = W_o (sum_{j <= t} g_j l_j) / (t + 1)."""
import json
import os

import pytest
import torch

from tests.plain import llama_plain as plain
from tests.util import max_rel_diff

pytestmark = pytest.mark.gpu
NAME = "ToyLatentCache"
LATENT, GATE_W = 12, 3


def _register():
    from dataclasses import dataclass
    from vllm_oxide_b200.config import Architecture, register_architecture
    from vllm_oxide_b200.parts import Block, CacheSpec, Embedding, LayerCall, LMHead, Mixer, ModelSpec, RMSNorm, SwiGLU
    from vllm_oxide_b200.parts.base import PagedTensorSpec
    from vllm_oxide_b200.weights import TensorSpec

    @dataclass(frozen=True)
    class ToyConfig:
        hidden: int
        inter: int
        layers: int
        vocab: int
        eps: float

        @classmethod
        def from_dict(cls, d, where="config.json"):
            return cls(d["toy_hidden"], d["toy_inter"], d["toy_layers"], d["toy_vocab"], d["toy_eps"])

        def to_dict(self):
            return {"architectures": [NAME], "toy_hidden": self.hidden, "toy_inter": self.inter, "toy_layers": self.layers,
                    "toy_vocab": self.vocab, "toy_eps": self.eps}

    class LatentMix(Mixer):
        def __init__(self, w_l, w_g, w_o, dtype, device):
            self.w_l = w_l.to(device=device, dtype=torch.float32)       # [LATENT, hidden]
            self.w_g = w_g.to(device=device, dtype=torch.float32)       # [GATE_W, hidden]; only its first row gates
            self.w_o = w_o.to(device=device, dtype=torch.float32)       # [hidden, LATENT]
            self.dtype = dtype

        def cache_spec(self):
            # two tensors per page, of different widths and dtypes: nothing like a key / value pair
            return CacheSpec(tensors=(PagedTensorSpec(1, LATENT), PagedTensorSpec(1, GATE_W, torch.float32)))

        def forward(self, x, ctx, cache, state, out=None):
            lat, gate = cache.tensors
            assert lat.shape[1:] == (1, cache.page_size, LATENT) and gate.shape[1:] == (1, cache.page_size, GATE_W)
            assert lat.dtype == self.dtype and gate.dtype == torch.float32
            ps = cache.page_size
            T = x.shape[0]
            xf = x.float()
            l_new = (xf @ self.w_l.t()).to(self.dtype)
            g_new = torch.sigmoid(xf @ self.w_g.t())
            slots = ctx.slot_mapping[cache.group][:T].long()
            real = slots >= 0
            lat[slots[real] // ps, 0, slots[real] % ps] = l_new[real]
            gate[slots[real] // ps, 0, slots[real] % ps] = g_new[real]
            res = torch.zeros(T, self.w_o.shape[0], dtype=torch.float32, device=x.device)
            starts, ctxs = ctx.seq_starts.tolist(), ctx.context_lens.tolist()
            table = ctx.block_tables[cache.group]
            for s in range(ctx.seqs):
                r0, r1 = starts[s], starts[s + 1]
                if r1 <= r0:
                    continue
                n = ctxs[s] + (r1 - r0)                                    # keys after this step, all read from the pages
                pages = table[s, :-(-n // ps)].long()
                l_all = lat[pages, 0].reshape(-1, LATENT)[:n].float()
                g_all = gate[pages, 0].reshape(-1, GATE_W)[:n, :1]
                csum = torch.cumsum(g_all * l_all, 0)[ctxs[s]:]
                cnt = torch.arange(ctxs[s] + 1, n + 1, device=x.device, dtype=torch.float32)[:, None]
                res[r0:r1] = (csum / cnt) @ self.w_o.t()
            return res.to(self.dtype)

    def manifest(c):
        m = {"emb": TensorSpec((c.vocab, c.hidden)), "final": TensorSpec((c.hidden,), init="ones")}
        for i in range(c.layers):
            m[f"l{i}.wl"] = TensorSpec((LATENT, c.hidden))
            m[f"l{i}.wg"] = TensorSpec((GATE_W, c.hidden))
            m[f"l{i}.wo"] = TensorSpec((c.hidden, LATENT))
            m[f"l{i}.n1"] = TensorSpec((c.hidden,), init="ones")
            m[f"l{i}.n2"] = TensorSpec((c.hidden,), init="ones")
            m[f"l{i}.gate"] = TensorSpec((c.inter, c.hidden))
            m[f"l{i}.up"] = TensorSpec((c.inter, c.hidden))
            m[f"l{i}.down"] = TensorSpec((c.hidden, c.inter))
        return m

    def build(c, w, ctx):
        emb = Embedding(w.take("emb"), ctx.dtype, ctx.device)
        blocks = [Block(RMSNorm(w.take(f"l{i}.n1"), c.eps, ctx.device),
                        LatentMix(w.take(f"l{i}.wl"), w.take(f"l{i}.wg"), w.take(f"l{i}.wo"), ctx.dtype, ctx.device),
                        RMSNorm(w.take(f"l{i}.n2"), c.eps, ctx.device),
                        SwiGLU(w.take(f"l{i}.gate"), w.take(f"l{i}.up"), w.take(f"l{i}.down"), ctx.dtype, ctx.device))
                  for i in range(c.layers)]
        spec = ModelSpec(embedding=emb, blocks=blocks, schedule=[LayerCall(i, i) for i in range(c.layers)],
                         final_norm=RMSNorm(w.take("final"), c.eps, ctx.device), lm_head=LMHead(emb.table),
                         hidden_size=c.hidden, vocab_size=c.vocab)
        w.finish()
        return spec

    register_architecture(Architecture(NAME, ToyConfig, manifest, build), replace=True)
    return ToyConfig


def _plain_logits(model_dir, tokens):
    """The toy model, whole sequence, float64, written out directly."""
    from safetensors.torch import load_file
    c = json.load(open(os.path.join(model_dir, "config.json")))
    t = {k: v.double() for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items()}
    x = plain.embedding(t["emb"], tokens)
    n = torch.arange(1, len(tokens) + 1, dtype=torch.float64)[:, None]
    for i in range(c["toy_layers"]):
        h = plain.rms_norm(x, t[f"l{i}.n1"], c["toy_eps"])
        lat = h @ t[f"l{i}.wl"].t()
        g = torch.sigmoid(h @ t[f"l{i}.wg"].t())[:, :1]
        x = x + (torch.cumsum(g * lat, 0) / n) @ t[f"l{i}.wo"].t()
        x = x + plain.feed_forward(plain.rms_norm(x, t[f"l{i}.n2"], c["toy_eps"]), t[f"l{i}.gate"], t[f"l{i}.up"], t[f"l{i}.down"])
    return plain.linear(plain.rms_norm(x, t["final"], c["toy_eps"]), t["emb"])


def test_a_cache_that_is_no_key_value_pair_runs_through_the_unchanged_framework(tmp_path):
    from vllm_oxide_b200.config import EngineConfig, unregister_architecture
    from vllm_oxide_b200.engine import LLM, ModelRunner
    from vllm_oxide_b200.replay.trace import TraceSession
    from vllm_oxide_b200.sampling import SamplingParams
    from vllm_oxide_b200.weights import write_random_model
    ToyConfig = _register()
    try:
        d = str(tmp_path / "toy")
        write_random_model(d, ToyConfig(24, 40, 2, 61, 1e-5), seed=9, std=0.3, norm_jitter=0.2)
        page = 8
        eng = EngineConfig(max_batch_tokens=64, max_seqs=4, max_model_len=64, block_size=page, num_pages=10, dtype="float32",
                           cuda_graphs=False)
        runner = ModelRunner.from_dir(d, eng)
        pools = runner.pools
        assert pools.num_groups == 1 and len(pools.kv) == 2
        assert [tuple(t.shape) for t in pools.kv[0]] == [(10, 1, page, LATENT), (10, 1, page, GATE_W)]
        assert pools.kv[0][0].dtype == torch.float32 and pools.kv[0][1].dtype == torch.float32
        assert pools.bytes_per_token() == 2 * (LATENT * 4 + GATE_W * 4)          # two layers
        for ts in pools.kv.values():                                               # stale contents must never be read
            for t in ts:
                t.fill_(float("nan"))
        s = TraceSession(runner)
        reqs = {"a": [(5 * i + 1) % 61 for i in range(37)], "b": [(3 * i + 7) % 61 for i in range(20)]}
        want = {k: _plain_logits(d, v) for k, v in reqs.items()}
        whole = s.run_step({"step": 0, "entries": [{"id": "a", "tokens": reqs["a"], "want": list(range(37))}], "end": ["a"]})
        assert max_rel_diff(whole, want["a"]) <= 2e-5
        # portions of both requests side by side, down to single tokens, over pages that were just given back
        cuts = {"a": [4, 9, 1, 16, 7], "b": [2, 2, 12, 1, 3]}
        pos, got = {"a": 0, "b": 0}, {"a": [], "b": []}
        for i in range(5):
            entries = [{"id": k, "tokens": reqs[k][pos[k]:pos[k] + cuts[k][i]], "want": list(range(cuts[k][i]))} for k in ("a", "b")]
            out = s.run_step({"step": 1 + i, "entries": entries, "end": []})
            got["a"].append(out[:cuts["a"][i]])
            got["b"].append(out[cuts["a"][i]:])
            for k in pos:
                pos[k] += cuts[k][i]
        for k in reqs:
            assert max_rel_diff(torch.cat(got[k]), want[k]) <= 2e-5
        s.run_step({"step": 9, "entries": [], "end": ["a", "b"]})
        assert runner.manager.num_free_pages(0) == 10 and runner.manager.check_invariants() == ""
        # generation over the scheduler: a pool of 10 pages for four requests that grow: someone is preempted and recomputed
        llm = LLM(runner)
        prompts = [reqs["a"][:14], reqs["b"][:9], reqs["a"][3:20], reqs["b"][:5]]
        outs = llm.generate(prompts, SamplingParams(max_new_tokens=10, stop_token_ids=()))
        for prompt, o in zip(prompts, outs):
            seq = list(prompt)
            for tok in o.token_ids:
                assert tok == int(_plain_logits(d, seq)[-1].argmax())
                seq.append(tok)
        assert llm.stats["preemptions"] > 0
        assert runner.manager.num_free_pages(0) == 10 and runner.manager.check_invariants() == ""
    finally:
        unregister_architecture(NAME)
