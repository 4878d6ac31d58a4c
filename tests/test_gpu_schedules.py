"""The schedules the benchmark itself runs, compared with the plain implementation: decode steps of
12 to 64 live requests (the folded five-kernel path up to 32 rows, the many-row path above it, the
decode attention kernel at 64 rows), the same through `LLM.generate` with CUDA graphs of batch
classes 16 / 32 / 64 and steps launched ahead, a mixed step of dozens of single tokens beside a
portion that fills the 2,048-token budget, and a whole 2,048-token prompt in one step at the
benchmark's layer widths. In 32-bit and in bfloat16 (the reference's batch-invariance and
chunking tests, crates/engine/src/model.rs:450-584, at these sizes)."""
import pytest
import torch

from tests.test_gpu_generate import assert_same_or_near_tie, sp
from tests.test_gpu_replay import _session, check, oracle, run_trace
from tests.util import TINY, TOL, make_model_dir, max_rel_diff, random_tokens

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]
BATCHES = (12, 32, 33, 48, 64)


def _pack(pending, budget):
    """Cut a list of (name, tokens) into steps of whole prompts under a token budget."""
    steps, cur, used = [], [], 0
    for name, toks in pending:
        if cur and used + len(toks) > budget:
            steps.append(cur)
            cur, used = [], 0
        cur.append((name, toks))
        used += len(toks)
    if cur:
        steps.append(cur)
    return steps


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", ["D", "1Bv"])
def test_decode_steps_of_12_to_64_live_requests(tmp_path_factory, name, dtype):
    """64 requests with contexts of 14 to 80 tokens are prefilled; then, for each batch size, two
    steps in which the first so many requests bring one token each (the others are left out and
    go on later). Every row's logits are compared. Contexts differ and cross page edges on the way."""
    cfg, _, page = TINY[name]
    model_dir = make_model_dir(tmp_path_factory.getbasetemp(), name)
    per_batch = 2
    base = [14 + (5 * i) % 67 for i in range(64)]
    extra = [per_batch * sum(1 for b in BATCHES if i < b) for i in range(64)]
    reqs = {f"q{i}": random_tokens(base[i] + extra[i], cfg.vocab_size, 3000 + i) for i in range(64)}
    assert any((base[i] + k) % page == 0 for i in range(64) for k in range(extra[i]))      # a page's edge is crossed while decoding
    s = _session(model_dir, dtype, 64 * 96, page, max_seqs=64, max_batch_tokens=2048, max_model_len=128)
    steps, n = [], 0
    for group in _pack([(f"q{i}", reqs[f"q{i}"][:base[i]]) for i in range(64)], 2048):
        steps.append({"step": n, "entries": [{"id": nm, "tokens": t, "want": [len(t) - 1]} for nm, t in group], "end": []})
        n += 1
    pos = list(base)
    for b in BATCHES:
        for _ in range(per_batch):
            steps.append({"step": n, "entries": [{"id": f"q{i}", "tokens": [reqs[f"q{i}"][pos[i]]], "want": [0]} for i in range(b)],
                          "end": []})
            for i in range(b):
                pos[i] += 1
            n += 1
    assert pos == [len(reqs[f"q{i}"]) for i in range(64)]
    steps[-1]["end"] = list(reqs)
    worst = check(run_trace(s, steps), model_dir, reqs, dtype, "decode steps of many requests")
    assert s.runner.manager.check_invariants() == ""
    assert s.runner.manager.num_free_pages(0) == s.runner.manager.num_pages(0)
    print(f"{name} {dtype}: decode steps of {BATCHES} requests, worst rel diff {worst:.2e}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["D", "1Bv"])
def test_generation_of_64_requests_with_graphs_and_steps_ahead(tmp_path_factory, name, dtype):
    """64 requests at once through `LLM.generate`; they end at different lengths, so the decode
    steps pass through the batch classes 64, 32 and 16 of the recorded graphs. Tokens are those of
    steps launched one by one (float32: exactly; bfloat16: up to near-ties of the oracle's logits)."""
    from vllm_oxide_b200.engine import LLM
    cfg, _, page = TINY[name]
    model_dir = make_model_dir(tmp_path_factory.getbasetemp(), name)
    prompts = [random_tokens(9 + (11 * i) % 50, cfg.vocab_size, 5000 + i) for i in range(64)]
    params = [sp(max_new_tokens=5 + 7 * (i % 4) + (1 if i >= 60 else 0), temperature=0.0 if i % 5 else 0.6, seed=i, stop_token_ids=())
              for i in range(64)]
    kw = dict(max_batch_tokens=2048, max_seqs=64, max_model_len=128, block_size=page, num_pages=64 * 128 // page)
    want = LLM(model_dir, dtype=dtype, cuda_graphs=False, **kw).generate(prompts, params)
    llm = LLM(model_dir, dtype=dtype, cuda_graphs=True, run_ahead=True, **kw)
    got = llm.generate(prompts, params)
    classes = {key[0] for key in llm.runner._graphs}
    assert {16, 32, 64} <= classes, classes
    assert llm.stats["ahead_steps"] > 0 and llm.stats["graph_steps"] > 0
    tol = 0.0 if dtype == "float32" else TOL[torch.bfloat16]
    for p, prm, g, w in zip(prompts, params, got, want):
        assert len(g.token_ids) == prm.max_new_tokens
        assert_same_or_near_tie(model_dir, p, g.token_ids, w.token_ids, prm, tol)
    # and against the plain implementation itself: the first token of some of the greedy requests
    for p, prm, g in list(zip(prompts, params, got))[::3]:
        if prm.temperature == 0.0:
            ref = oracle(model_dir, p)[-1]
            pick = int(ref.argmax())
            assert g.token_ids[0] == pick or float(ref[pick] - ref[g.token_ids[0]]) <= (tol or 1e-5) * float(ref.abs().max())
    assert llm.runner.manager.check_invariants() == ""
    assert llm.runner.manager.num_free_pages(0) == llm.runner.manager.num_pages(0)


def _long_request(cfg, n=2048):
    return random_tokens(n, cfg.vocab_size, 777)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", ["D", "1Bv"])
def test_mixed_step_of_40_single_tokens_beside_a_full_portion(tmp_path_factory, name, dtype):
    """The serving run's steady state: 40 decoding requests lead the batch with one token each and
    one portion of a long prompt fills what is left of the 2,048-token budget; the next step
    brings the same 40 beside the prompt's short rest. Logits of every single token and of the
    portions' ends (and of the rest's every row) are compared."""
    cfg, _, page = TINY[name]
    model_dir = make_model_dir(tmp_path_factory.getbasetemp(), name)
    singles = {f"s{i}": random_tokens(20 + (3 * i) % 41 + 2, cfg.vocab_size, 8000 + i) for i in range(40)}
    long_toks = _long_request(cfg)
    reqs = dict(singles, long=long_toks)
    s = _session(model_dir, dtype, 2048 + 64 + 40 * 80, page, max_seqs=64, max_batch_tokens=2048, max_model_len=2048 + 64)
    steps, n = [], 0
    for group in _pack([(nm, t[:-2]) for nm, t in singles.items()], 2048):
        steps.append({"step": n, "entries": [{"id": nm, "tokens": t, "want": [len(t) - 1]} for nm, t in group], "end": []})
        n += 1
    first = 2048 - 40
    steps.append({"step": n, "entries": [{"id": nm, "tokens": [t[-2]], "want": [0]} for nm, t in singles.items()]
                  + [{"id": "long", "tokens": long_toks[:first], "want": [0, first // 2, first - 1]}], "end": []})
    steps.append({"step": n + 1, "entries": [{"id": nm, "tokens": [t[-1]], "want": [0]} for nm, t in singles.items()]
                  + [{"id": "long", "tokens": long_toks[first:], "want": list(range(2048 - first))}], "end": list(reqs)})
    assert sum(len(e["tokens"]) for e in steps[-2]["entries"]) == 2048
    worst = check(run_trace(s, steps), model_dir, reqs, dtype, "40 single tokens beside a portion")
    assert s.runner.manager.num_free_pages(0) == s.runner.manager.num_pages(0)
    print(f"{name} {dtype}: mixed step, worst rel diff {worst:.2e}")


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_whole_2048_token_prompt_in_one_step_at_the_benchmark_widths(tmp_path_factory, dtype):
    """The timed prefill's path: 2,048 rows in one step at Llama 3.2 1B's layer widths (the two-SM
    gate/up product with SwiGLU at N = 16,384, tcgen05 attention over 16 row tiles, the many-row
    products), logits at the first, a middle and the last row; then the last 32 tokens once more,
    one by one, from the cache that step left."""
    cfg, _, page = TINY["1Bv"]
    model_dir = make_model_dir(tmp_path_factory.getbasetemp(), "1Bv")
    toks = _long_request(cfg)
    reqs = {"long": toks}
    s = _session(model_dir, dtype, 2048 + 64, page, max_seqs=4, max_batch_tokens=2048)
    whole = [{"step": 0, "entries": [{"id": "long", "tokens": toks, "want": [0, 1023, 2047]}], "end": ["long"]}]
    w1 = check(run_trace(s, whole), model_dir, reqs, dtype, "2,048 tokens in one step")
    cut = 2048 - 32
    tail = [{"step": 1, "entries": [{"id": "long", "tokens": toks[:cut], "want": [cut - 1]}], "end": []}]
    tail += [{"step": 2 + i, "entries": [{"id": "long", "tokens": [toks[cut + i]], "want": [0]}], "end": ["long"] if i == 31 else []}
             for i in range(32)]
    w2 = check(run_trace(s, tail), model_dir, reqs, dtype, "2,016 tokens, then 32 one by one")
    assert s.runner.manager.num_free_pages(0) == s.runner.manager.num_pages(0)
    print(f"1B widths {dtype}: 2,048-token step worst rel diff {w1:.2e}, bulk + 32 single tokens {w2:.2e}")


def test_2048_token_prefill_replayed_from_a_graph_picks_the_plain_token(tmp_path_factory):
    """The same prompt three times through `LLM.generate` in bfloat16: the step is launched kernel
    by kernel, recorded at its second sighting and replayed at the third. Each time the first token
    is the plain implementation's pick (or a near-tie of it), and the replayed run equals the others."""
    from vllm_oxide_b200.engine import LLM
    cfg, _, page = TINY["1Bv"]
    model_dir = make_model_dir(tmp_path_factory.getbasetemp(), "1Bv")
    toks = _long_request(cfg)
    llm = LLM(model_dir, dtype="bfloat16", max_batch_tokens=2048, max_seqs=4, max_model_len=2048 + 64, block_size=page,
              num_pages=(2048 + 64) // page + 4, step_graphs=2)
    params = sp(max_new_tokens=3, stop_token_ids=())
    runs = [llm.generate([toks], params)[0].token_ids for _ in range(3)]
    assert llm.runner.step_graph_replays >= 1
    ref = oracle(model_dir, toks)[-1]
    pick = int(ref.argmax())
    for r in runs:
        assert r[0] == pick or float(ref[pick] - ref[r[0]]) <= TOL[torch.bfloat16] * float(ref.abs().max())
    for r in runs[1:]:
        assert_same_or_near_tie(model_dir, toks, r, runs[0], params, TOL[torch.bfloat16])
