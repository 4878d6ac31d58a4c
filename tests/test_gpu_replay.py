"""Trace replay against the plain implementation, in 32-bit and in bfloat16: whole requests,
bulk + 32 single tokens, portions of changing size down to two tokens, and mixed batches of up to
four live requests over a pool so small that pages are used again."""
import json
import os
import random
import subprocess
import sys

import pytest
import torch

from tests.plain import llama_plain as plain
from tests.util import TINY, TOL, make_model_dir, max_rel_diff, random_tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _session(model_dir, dtype, max_tokens, page, max_seqs=8, max_batch_tokens=None, max_model_len=None):
    from vllm_oxide_b200.config import EngineConfig
    from vllm_oxide_b200.engine import ModelRunner
    from vllm_oxide_b200.replay.trace import TraceSession
    pages = -(-max_tokens // page)
    eng = EngineConfig(max_batch_tokens=max_batch_tokens or pages * page, max_seqs=max_seqs, max_model_len=max_model_len or pages * page,
                       block_size=page, num_pages=pages, dtype=dtype, cuda_graphs=False)
    return TraceSession(ModelRunner.from_dir(model_dir, eng))


_oracle_cache = {}


def oracle(model_dir, tokens):
    key = (model_dir, tuple(tokens))
    if key not in _oracle_cache:
        cfg, tensors = plain.load_model(model_dir)
        _oracle_cache[key] = plain.forward(cfg, tensors, list(tokens))
    return _oracle_cache[key]


def run_trace(session, steps):
    """Replay; returns {(request, position): logits row}."""
    got = {}
    pos = {}
    for msg in steps:
        out = session.run_step(msg)
        r = 0
        for e in msg["entries"]:
            base = pos.get(e["id"], 0)
            for w in e.get("want", []):
                got[(e["id"], base + w)] = out[r]
                r += 1
            pos[e["id"]] = base + len(e["tokens"])
        for name in msg.get("end", []):
            pos.pop(name, None)
        assert (out is None and r == 0) or out.shape[0] == r
    return got


def check(got, model_dir, requests, dtype, what):
    worst = 0.0
    for name, toks in requests.items():
        ref = oracle(model_dir, toks)
        rows = [p for (n, p) in got if n == name]
        assert rows, f"{what}: no logits for {name}"
        for p in rows:
            d = max_rel_diff(got[(name, p)], ref[p])
            assert d <= TOL[dtype], f"{what}: request {name} position {p}: rel diff {d:.3e} > {TOL[dtype]:.1e}"
            worst = max(worst, d)
    return worst


def whole_steps(requests):
    steps = []
    for i, (name, toks) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": name, "tokens": toks, "want": list(range(len(toks)))}], "end": [name]})
    return steps


def bulk_tail_steps(requests, tail=32):
    steps, n = [], 0
    for name, toks in requests.items():
        cut = max(1, len(toks) - tail)
        steps.append({"step": n, "entries": [{"id": name, "tokens": toks[:cut], "want": [cut - 1]}], "end": []})
        n += 1
        for p in range(cut, len(toks)):
            steps.append({"step": n, "entries": [{"id": name, "tokens": [toks[p]], "want": [0]}],
                          "end": [name] if p == len(toks) - 1 else []})
            n += 1
        if cut == len(toks):
            steps[-1]["end"] = [name]
    return steps


def portion_steps(requests, sizes=(16, 7, 2, 5, 3, 11, 2, 1, 9)):
    steps, n = [], 0
    for name, toks in requests.items():
        p, k = 0, 0
        while p < len(toks):
            c = min(sizes[k % len(sizes)], len(toks) - p)
            k += 1
            steps.append({"step": n, "entries": [{"id": name, "tokens": toks[p:p + c], "want": list(range(c))}],
                          "end": [name] if p + c == len(toks) else []})
            p += c
            n += 1
    return steps


def mixed_steps(requests, seed, live_max=4):
    """Up to four live requests; each step gives some of them a portion (2..16 tokens while far from
    their end, single tokens for their last 12) and leaves some out; finished ones end and the
    next request takes their pages."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live = {}
    steps, n = [], 0
    while waiting or live:
        while waiting and len(live) < live_max:
            name, toks = waiting.pop(0)
            live[name] = [toks, 0]
        entries, ends = [], []
        for name in list(live):
            toks, p = live[name]
            if len(live) > 1 and rng.random() < 0.25:
                continue                                  # left out of this step, goes on later
            left = len(toks) - p
            c = 1 if left <= 12 else min(left - 12, rng.choice([2, 3, 5, 8, 16]))
            entries.append({"id": name, "tokens": toks[p:p + c], "want": list(range(c))})
            live[name][1] = p + c
            if p + c == len(toks):
                ends.append(name)
                del live[name]
        if entries:
            steps.append({"step": n, "entries": entries, "end": ends})
            n += 1
    return steps


def _requests(vocab, lengths, seed):
    return {f"r{i}": random_tokens(L, vocab, seed + i) for i, L in enumerate(lengths)}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_four_ways_of_cutting(tmp_path_factory, name, dtype):
    cfg, _, page = TINY[name]
    model_dir = make_model_dir(tmp_path_factory.getbasetemp(), name)
    lengths = {"A": [5, 17, 33, 100], "B": [1, 9, 40, 70], "C": [3, 64, 65, 90], "D": [2, 63, 64, 127]}[name]
    reqs = _requests(cfg.vocab_size, lengths, 100)
    s = _session(model_dir, dtype, 128, page)
    w1 = check(run_trace(s, whole_steps(reqs)), model_dir, reqs, dtype, "whole")
    w2 = check(run_trace(s, bulk_tail_steps(reqs)), model_dir, reqs, dtype, "bulk+tail")
    w3 = check(run_trace(s, portion_steps(reqs)), model_dir, reqs, dtype, "portions")
    assert s.runner.manager.check_invariants() == ""
    assert s.runner.manager.num_free_pages(0) == s.runner.manager.num_pages(0)
    print(f"{name} {dtype}: worst rel diff whole {w1:.2e} bulk+tail {w2:.2e} portions {w3:.2e}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_mixed_batches_reuse_pages(tmp_path_factory, name, dtype):
    cfg, _, page = TINY[name]
    model_dir = make_model_dir(tmp_path_factory.getbasetemp(), name)
    lengths = [60, 23, 64, 41, 17, 50, 33, 2, 58]
    reqs = _requests(cfg.vocab_size, lengths, 500)
    # four live requests of at most 64 tokens: a pool of 256 tokens, every page taken again and again
    s = _session(model_dir, dtype, 256, page)
    steps = mixed_steps(reqs, seed=7)
    assert max(len(m["entries"]) for m in steps) == 4
    assert any(min(len(e["tokens"]) for e in m["entries"]) == 1 and max(len(e["tokens"]) for e in m["entries"]) > 1
               for m in steps), "the trace must put portions beside single tokens in one step"
    worst = check(run_trace(s, steps), model_dir, reqs, dtype, "mixed")
    assert s.runner.manager.check_invariants() == ""
    assert s.runner.manager.num_free_pages(0) == s.runner.manager.num_pages(0)
    print(f"{name} {dtype}: mixed worst rel diff {worst:.2e}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_four_ways_at_the_benchmark_layer_sizes(tmp_path_factory, dtype):
    """Two layers of Llama 3.2 1B's sizes (vocabulary 128256, 32 heads on 8 kv heads, K = 8192 in the
    down projection): the kernels at the sizes the benchmark runs, cut four ways. The longer request
    spans several row tiles and key tiles of the attention kernels."""
    cfg, _, page = TINY["1B"]
    model_dir = make_model_dir(tmp_path_factory.getbasetemp(), "1B")
    reqs = _requests(cfg.vocab_size, [150, 70], 77)
    s = _session(model_dir, dtype, 256, page)
    w1 = check(run_trace(s, whole_steps(reqs)), model_dir, reqs, dtype, "whole")
    w2 = check(run_trace(s, bulk_tail_steps(reqs)), model_dir, reqs, dtype, "bulk+tail")
    w3 = check(run_trace(s, portion_steps(reqs, sizes=(64, 7, 2, 33, 3, 16, 2, 1, 40))), model_dir, reqs, dtype, "portions")
    w4 = check(run_trace(s, mixed_steps(reqs, seed=11)), model_dir, reqs, dtype, "mixed")
    assert s.runner.manager.check_invariants() == ""
    assert s.runner.manager.num_free_pages(0) == s.runner.manager.num_pages(0)
    print(f"1B sizes {dtype}: worst rel diff whole {w1:.2e} bulk+tail {w2:.2e} portions {w3:.2e} mixed {w4:.2e}")


def test_four_ways_at_head_size_128(tmp_path_factory):
    """Head size 128 with three heads per kv head at a real width (hidden 3072): the tcgen05
    portion kernel's second instantiation and the decode kernel's, inside the engine, cut four ways."""
    dtype = torch.bfloat16
    cfg, _, page = TINY["HD128"]
    model_dir = make_model_dir(tmp_path_factory.getbasetemp(), "HD128")
    reqs = _requests(cfg.vocab_size, [170, 45], 31)
    s = _session(model_dir, dtype, 320, page)
    w1 = check(run_trace(s, whole_steps(reqs)), model_dir, reqs, dtype, "whole")
    w2 = check(run_trace(s, bulk_tail_steps(reqs)), model_dir, reqs, dtype, "bulk+tail")
    w3 = check(run_trace(s, portion_steps(reqs, sizes=(64, 7, 2, 33, 3, 16, 2, 1, 40))), model_dir, reqs, dtype, "portions")
    w4 = check(run_trace(s, mixed_steps(reqs, seed=5)), model_dir, reqs, dtype, "mixed")
    assert s.runner.manager.num_free_pages(0) == s.runner.manager.num_pages(0)
    print(f"head size 128: worst rel diff whole {w1:.2e} bulk+tail {w2:.2e} portions {w3:.2e} mixed {w4:.2e}")


def test_mixed_step_sends_leading_single_tokens_to_the_decode_kernel(tmp_path_factory, monkeypatch):
    """A mixed step whose first requests bring one token each: those rows go to the decode
    attention kernel, the portions behind them (and a single token that follows a portion) to the
    portion kernel. Same logits as the plain implementation either way."""
    from vllm_oxide_b200 import kernels
    dtype = torch.bfloat16
    cfg, _, page = TINY["D"]
    model_dir = make_model_dir(tmp_path_factory.getbasetemp(), "D")
    reqs = _requests(cfg.vocab_size, [90, 70, 100, 40, 33], 500)
    t = reqs
    calls = []
    real = kernels.attn_decode_mma
    monkeypatch.setattr(kernels, "attn_decode_mma", lambda q, *a, **k: (calls.append(q.shape[0]), real(q, *a, **k))[1])
    for split in (True, False):
        s = _session(model_dir, dtype, 448, page)
        for blk in s.runner.spec.blocks:
            blk.mixer.split_mixed = split
        steps = [
            {"step": 0, "entries": [{"id": "r0", "tokens": t["r0"][:80], "want": [79]}, {"id": "r1", "tokens": t["r1"][:69], "want": []},
                                    {"id": "r3", "tokens": t["r3"][:30], "want": [29]}], "end": []},
            {"step": 1, "entries": [{"id": "r0", "tokens": t["r0"][80:81], "want": [0]}, {"id": "r1", "tokens": t["r1"][69:70], "want": [0]},
                                    {"id": "r2", "tokens": t["r2"][:57], "want": [0, 56]}, {"id": "r3", "tokens": t["r3"][30:31], "want": [0]},
                                    {"id": "r4", "tokens": t["r4"], "want": [32]}], "end": ["r1", "r4"]},
            {"step": 2, "entries": [{"id": "r0", "tokens": t["r0"][81:82], "want": [0]}, {"id": "r3", "tokens": t["r3"][31:32], "want": [0]},
                                    {"id": "r2", "tokens": t["r2"][57:], "want": [42]}], "end": ["r0", "r2", "r3"]},
        ]
        calls.clear()
        check(run_trace(s, steps), model_dir, reqs, dtype, f"leading single tokens, split={split}")
        layers = cfg.num_hidden_layers
        assert calls == ([2] * layers + [2] * layers if split else []), calls
        assert s.runner.manager.num_free_pages(0) == s.runner.manager.num_pages(0)


def test_long_context_beside_a_short_one(tmp_path_factory):
    """Decode steps of a request of more than 6,144 keys beside a short one: the decode attention
    then shares a request's keys over up to 64 blocks that merge through global memory, and the
    short request uses only as many of them as it has keys for."""
    dtype = torch.bfloat16
    cfg, _, page = TINY["DL"]
    model_dir = make_model_dir(tmp_path_factory.getbasetemp(), "DL")
    reqs = _requests(cfg.vocab_size, [6300, 150], 900)
    s = _session(model_dir, dtype, 6336 + 192, page)
    steps, n = [], 0
    long_toks, short_toks = reqs["r0"], reqs["r1"]
    for lo in range(0, 6280, 2048):
        hi = min(lo + 2048, 6280)
        steps.append({"step": n, "entries": [{"id": "r0", "tokens": long_toks[lo:hi], "want": [hi - lo - 1]}], "end": []})
        n += 1
    steps.append({"step": n, "entries": [{"id": "r1", "tokens": short_toks[:130], "want": [129]}], "end": []})
    n += 1
    for i in range(20):
        steps.append({"step": n, "entries": [{"id": "r0", "tokens": [long_toks[6280 + i]], "want": [0]},
                                             {"id": "r1", "tokens": [short_toks[130 + i]], "want": [0]}],
                      "end": ["r0", "r1"] if i == 19 else []})
        n += 1
    from vllm_oxide_b200.tuning import TUNING
    LONG_CONTEXT_KEYS = TUNING.long_context_keys
    assert LONG_CONTEXT_KEYS < 6280
    worst = check(run_trace(s, steps), model_dir, reqs, dtype, "long beside short")
    assert s.runner.manager.num_free_pages(0) == s.runner.manager.num_pages(0)
    print(f"long context: worst rel diff {worst:.2e}")


@pytest.mark.parametrize("name", ["D", "1Bv"])
def test_a_wrong_page_in_one_layer_is_seen_in_bfloat16(tmp_path_factory, name):
    """What the bfloat16 tolerance cannot hide: the traces above run once more while ONE layer's
    attention reads a wrong page in place of one of the request's own (its third page where the
    second should be; the cache itself is right, the other layers read it rightly). Rows that see
    that page then differ from the plain implementation by more than the tolerance the tests allow,
    for a portion kernel's rows and for the decode kernel's alike: a fault of that kind fails the
    bfloat16 tests, not only the 32-bit ones. (Pages in swapped ORDER would not show in rows behind
    them: a softmax-weighted sum does not depend on the order of its keys.)"""
    dtype = torch.bfloat16
    cfg, _, page = TINY[name]
    model_dir = make_model_dir(tmp_path_factory.getbasetemp(), name)
    reqs = _requests(cfg.vocab_size, [127], 100)
    s = _session(model_dir, dtype, 128, page)
    mixer = s.runner.spec.blocks[-1].mixer
    attend = mixer.attend

    def swapped(q, out, ctx, cache):
        bt = ctx.block_tables[cache.group]
        keep = bt[:, 1].clone()
        bt[:, 1] = bt[:, 2]
        try:
            attend(q, out, ctx, cache)
        finally:
            bt[:, 1] = keep
    for what, steps in (("whole", whole_steps(reqs)), ("bulk+tail", bulk_tail_steps(reqs))):
        check(run_trace(s, steps), model_dir, reqs, dtype, what)          # the engine as it is: within the tolerance
        mixer.attend = swapped
        try:
            got = run_trace(s, steps)
        finally:
            mixer.attend = attend
        ref = oracle(model_dir, reqs["r0"])
        late = [max_rel_diff(got[k], ref[k[1]]) for k in got if k[1] >= 3 * page]
        print(f"{name} {what}: rows behind the wrong page differ by {min(late):.2e} .. {max(late):.2e} (tolerance {TOL[dtype]:.0e})")
        assert late and min(late) > TOL[dtype], f"{what}: a wrong page changed the logits by only {min(late):.2e}"


def test_f32_cuts_agree_closely(tmp_path_factory):
    """In 32-bit, the same position computed whole, token by token and in portions agrees far
    inside the tolerance against the oracle: the reference's bound between two of its own paths
    is 1e-5 relative (crates/engine/src/model.rs:492,536)."""
    cfg, _, page = TINY["B"]
    model_dir = make_model_dir(tmp_path_factory.getbasetemp(), "B")
    reqs = _requests(cfg.vocab_size, [70], 900)
    s = _session(model_dir, torch.float32, 128, page)
    a = run_trace(s, whole_steps(reqs))
    b = run_trace(s, portion_steps(reqs))
    c = run_trace(s, bulk_tail_steps(reqs))
    for k in a:
        if k in b:
            assert max_rel_diff(b[k], a[k]) <= 1e-5
        if k in c:
            assert max_rel_diff(c[k], a[k]) <= 1e-5


def test_trace_run_program(tmp_path):
    """bin/trace_run as a user runs it: JSON lines in, `done <step>` lines and .f32 files out."""
    cfg, _, page = TINY["A"]
    model_dir = make_model_dir(tmp_path, "A")
    reqs = _requests(cfg.vocab_size, [21, 40], 40)
    steps = mixed_steps(reqs, seed=3)
    out_dir = os.path.join(str(tmp_path), "out")
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype",
                           "float32", "--out", out_dir, "--max-tokens", "128"],
                          input="".join(json.dumps(m) + "\n" for m in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {m['step']}" for m in steps]
    pos = {}
    import numpy as np
    for m in steps:
        wanted = sum(len(e["want"]) for e in m["entries"])
        data = np.fromfile(os.path.join(out_dir, f"{m['step']}.f32"), dtype="<f4").reshape(wanted, cfg.vocab_size)
        r = 0
        for e in m["entries"]:
            ref = oracle(model_dir, reqs[e["id"]])
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                assert max_rel_diff(torch.from_numpy(data[r].copy()), ref[base + w]) <= TOL[torch.float32]
                r += 1
            pos[e["id"]] = base + len(e["tokens"])
