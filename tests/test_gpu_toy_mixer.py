"""A toy mixer with state of its own, defined here, is registered, built from a model folder and
stepped by the unchanged framework: configuration class, manifest, builder, state slots, portions
and mixed batches, generation with preemption. It is no model of anyone's: out[t] = W * mean(x[0..t])."""
import os

import pytest
import torch

from tests.util import max_rel_diff

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _register():
    from dataclasses import dataclass
    from vllm_oxide_b200.config import Architecture, register_architecture
    from vllm_oxide_b200.parts import (Block, Embedding, LayerCall, LMHead, Mixer, ModelSpec, RMSNorm, StateSpec, SwiGLU)
    from vllm_oxide_b200.parts.linear import to_compute
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
            return {"architectures": ["ToyRunningMean"], "toy_hidden": self.hidden, "toy_inter": self.inter,
                    "toy_layers": self.layers, "toy_vocab": self.vocab, "toy_eps": self.eps}

    class RunningMean(Mixer):
        """State per request: the sum of its inputs so far and their count."""

        def __init__(self, w, dtype, device):
            self.w = to_compute(w, torch.float32, device)
            self.h = w.shape[1]
            self.dtype = dtype

        def state_spec(self):
            return StateSpec((self.h + 1,), torch.float32)

        def forward(self, x, ctx, cache, state, out=None):
            assert cache is None and state is not None
            res = torch.empty(x.shape[0], self.h, dtype=torch.float32, device=x.device)
            slots = ctx.state_slots.tolist()
            starts = ctx.seq_starts.tolist()
            for s in range(ctx.seqs):
                r0, r1 = starts[s], starts[s + 1]
                st = state[slots[s]]
                csum = st[:self.h] + torch.cumsum(x[r0:r1].float(), 0)
                cnt = st[self.h] + torch.arange(1, r1 - r0 + 1, device=x.device, dtype=torch.float32)
                res[r0:r1] = (csum / cnt[:, None]) @ self.w.t()
                st[:self.h] = csum[-1]
                st[self.h] = cnt[-1]
            return res.to(self.dtype)          # a tensor of its own: the block copies it where it wants it

    def manifest(c):
        m = {"emb": TensorSpec((c.vocab, c.hidden)), "final": TensorSpec((c.hidden,), init="ones")}
        for i in range(c.layers):
            m[f"l{i}.mix"] = TensorSpec((c.hidden, c.hidden))
            m[f"l{i}.n1"] = TensorSpec((c.hidden,), init="ones")
            m[f"l{i}.n2"] = TensorSpec((c.hidden,), init="ones")
            m[f"l{i}.gate"] = TensorSpec((c.inter, c.hidden))
            m[f"l{i}.up"] = TensorSpec((c.inter, c.hidden))
            m[f"l{i}.down"] = TensorSpec((c.hidden, c.inter))
        return m

    def build(c, w, ctx):
        emb = Embedding(w.take("emb"), ctx.dtype, ctx.device)
        blocks = [Block(RMSNorm(w.take(f"l{i}.n1"), c.eps, ctx.device), RunningMean(w.take(f"l{i}.mix"), ctx.dtype, ctx.device),
                        RMSNorm(w.take(f"l{i}.n2"), c.eps, ctx.device),
                        SwiGLU(w.take(f"l{i}.gate"), w.take(f"l{i}.up"), w.take(f"l{i}.down"), ctx.dtype, ctx.device))
                  for i in range(c.layers)]
        spec = ModelSpec(embedding=emb, blocks=blocks, schedule=[LayerCall(i, None) for i in range(c.layers)],
                         final_norm=RMSNorm(w.take("final"), c.eps, ctx.device), lm_head=LMHead(emb.table),
                         hidden_size=c.hidden, vocab_size=c.vocab)
        w.finish()
        return spec

    register_architecture(Architecture("ToyRunningMean", ToyConfig, manifest, build), replace=True)
    return ToyConfig


def _plain_logits(model_dir, tokens):
    """The toy model, whole sequence, float64, written out directly."""
    import json
    from safetensors.torch import load_file
    from tests.plain import llama_plain as plain
    c = json.load(open(os.path.join(model_dir, "config.json")))
    t = {k: v.double() for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items()}
    x = plain.embedding(t["emb"], tokens)
    for i in range(c["toy_layers"]):
        n = plain.rms_norm(x, t[f"l{i}.n1"], c["toy_eps"])
        mean = torch.cumsum(n, 0) / torch.arange(1, len(tokens) + 1, dtype=torch.float64)[:, None]
        x = x + mean @ t[f"l{i}.mix"].t()
        x = x + plain.feed_forward(plain.rms_norm(x, t[f"l{i}.n2"], c["toy_eps"]), t[f"l{i}.gate"], t[f"l{i}.up"], t[f"l{i}.down"])
    return plain.linear(plain.rms_norm(x, t["final"], c["toy_eps"]), t["emb"])


def test_toy_stateful_mixer_runs_through_the_unchanged_framework(tmp_path):
    from vllm_oxide_b200.config import EngineConfig, unregister_architecture
    from vllm_oxide_b200.engine import LLM, ModelRunner
    from vllm_oxide_b200.replay.trace import TraceSession
    from vllm_oxide_b200.sampling import SamplingParams
    from vllm_oxide_b200.weights import write_random_model
    ToyConfig = _register()
    try:
        d = str(tmp_path / "toy")
        write_random_model(d, ToyConfig(24, 40, 2, 53, 1e-5), seed=4, std=0.3, norm_jitter=0.2)
        eng = EngineConfig(max_batch_tokens=64, max_seqs=3, max_model_len=64, block_size=8, num_pages=4, dtype="float32", cuda_graphs=False)
        runner = ModelRunner.from_dir(d, eng)
        assert runner.pools.num_groups == 0 and len(runner.pools.state) == 2          # no pages, two state tensors
        s = TraceSession(runner)
        reqs = {"a": [(5 * i + 1) % 53 for i in range(30)], "b": [(3 * i + 7) % 53 for i in range(17)]}
        want = {k: _plain_logits(d, v) for k, v in reqs.items()}
        whole = s.run_step({"step": 0, "entries": [{"id": "a", "tokens": reqs["a"], "want": list(range(30))}], "end": ["a"]})
        assert max_rel_diff(whole, want["a"]) <= 2e-5
        # portions of both requests side by side: the state is carried per request, in its slot
        cuts = {"a": [4, 9, 1, 16], "b": [2, 2, 12, 1]}
        pos, got = {"a": 0, "b": 0}, {"a": [], "b": []}
        for i in range(4):
            entries = [{"id": k, "tokens": reqs[k][pos[k]:pos[k] + cuts[k][i]], "want": list(range(cuts[k][i]))} for k in ("a", "b")]
            out = s.run_step({"step": 1 + i, "entries": entries, "end": []})
            got["a"].append(out[:cuts["a"][i]])
            got["b"].append(out[cuts["a"][i]:])
            for k in pos:
                pos[k] += cuts[k][i]
        for k in reqs:
            assert max_rel_diff(torch.cat(got[k]), want[k]) <= 2e-5
        s.run_step({"step": 9, "entries": [], "end": ["a", "b"]})
        # a slot that is used again starts from zero state
        again = s.run_step({"step": 10, "entries": [{"id": "c", "tokens": reqs["b"], "want": [16]}], "end": ["c"]})
        assert max_rel_diff(again[0], want["b"][16]) <= 2e-5
        # generation over the scheduler, more requests than state slots
        llm = LLM(runner)
        outs = llm.generate([reqs["a"][:6], reqs["b"][:9], reqs["a"][3:8], reqs["b"][:2]],
                            SamplingParams(max_new_tokens=5, stop_token_ids=()))
        for prompt, o in zip([reqs["a"][:6], reqs["b"][:9], reqs["a"][3:8], reqs["b"][:2]], outs):
            seq = list(prompt)
            for tok in o.token_ids:
                assert tok == int(_plain_logits(d, seq)[-1].argmax())
                seq.append(tok)
        assert runner.manager.num_free_slots() == 3
        # the same with the engine's defaults (CUDA graphs, steps launched ahead): this mixer reads
        # device data on the host, so no step of it can be recorded; the engine notices at its
        # first try, goes on launching steps one by one, and the tokens are the same
        eng2 = EngineConfig(max_batch_tokens=64, max_seqs=3, max_model_len=64, block_size=8, num_pages=4, dtype="float32")
        assert eng2.cuda_graphs and eng2.run_ahead
        llm2 = LLM(ModelRunner.from_dir(d, eng2))
        outs2 = llm2.generate([reqs["a"][:6], reqs["b"][:9], reqs["a"][3:8], reqs["b"][:2]],
                              SamplingParams(max_new_tokens=5, stop_token_ids=()))
        assert [o.token_ids for o in outs2] == [o.token_ids for o in outs]
        assert not llm2.runner.decode_graphs and not llm2.runner._graphs
    finally:
        unregister_architecture("ToyRunningMean")
