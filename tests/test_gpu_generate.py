"""Generation through the entry point: greedy against the plain implementation, batching and
preemption that leave a request's tokens unchanged, temperature sampling, long decoding, the first
tokens of a sequence, CUDA graphs on and off, and the errors of the reference's driver."""
import pytest
import torch

from tests.plain import llama_plain as plain
from tests.util import TINY, TOL, make_model_dir, max_rel_diff, random_tokens

pytestmark = pytest.mark.gpu


def llm_for(model_dir, dtype, page, **kw):
    from vllm_oxide_b200.engine import LLM
    args = dict(max_batch_tokens=64, max_seqs=8, max_model_len=256, block_size=page, num_pages=256 // page * 4)
    args.update(kw)
    return LLM(model_dir, dtype=dtype, **args)


def sp(**kw):
    from vllm_oxide_b200.sampling import SamplingParams
    return SamplingParams(**kw)


def assert_same_or_near_tie(model_dir, prompt, got, want, params, tol):
    """Two runs of one request must give the same tokens; in bfloat16 a difference is allowed only
    where it is a matter of rounding: at the first differing token both picks must be within
    `tol` (relative to the largest logit) of each other in the plain implementation's logits (with
    temperature sampling: in logit / temperature + noise). After such a near-tie the sequences
    differ legitimately and are not compared further."""
    if got == want:
        return
    assert tol > 0, f"tokens differ: {got} vs {want}"
    i = next(k for k in range(min(len(got), len(want))) if got[k] != want[k])
    pc, pt = plain.load_model(model_dir)
    logits = plain.forward(pc, pt, list(prompt) + list(want[:i]))[-1]
    scale = float(logits.abs().max())
    if params.temperature > 0:
        import numpy as np
        score = lambda t: float(logits[t]) / params.temperature + plain.gumbel_noise(params.seed, i, t)
        gap, scale = abs(score(got[i]) - score(want[i])), scale / params.temperature
    else:
        gap = abs(float(logits[got[i]]) - float(logits[want[i]]))
    assert gap <= tol * scale, f"token {i}: {got[i]} vs {want[i]} differ by {gap:.3e} of {scale:.3e}: more than rounding"


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_equals_plain_in_f32(tmp_path_factory, name):
    cfg, _, page = TINY[name]
    d = make_model_dir(tmp_path_factory.getbasetemp(), name)
    pc, pt = plain.load_model(d)
    llm = llm_for(d, "float32", page)
    from vllm_oxide_b200.engine import Generator
    gen = Generator(llm)
    lengths = {"A": [5, 17, 33], "B": [1, 9, 40]}[name]
    for i, L in enumerate(lengths):
        prompt = random_tokens(L, cfg.vocab_size, 10 + i)
        out = gen.greedy(prompt, 8, None, capture=(0, 1, 7))
        want = plain.greedy_generate(pc, pt, prompt, 8)
        assert out.tokens == want
        seq = prompt + want
        for gi, logits in out.captured:
            ref = plain.forward(pc, pt, seq[:L + gi])[-1]
            assert max_rel_diff(logits, ref) <= TOL[torch.float32]
        assert out.prefill_time > 0 and out.decode_time > 0
    # the same engine and pool serve call after call (crates/engine/src/generate.rs:165-173)
    assert llm.runner.manager.num_free_pages(0) == llm.runner.manager.num_pages(0)


def test_stop_token_is_kept_and_ends_the_output(tmp_path_factory):
    cfg, _, page = TINY["A"]
    d = make_model_dir(tmp_path_factory.getbasetemp(), "A")
    from vllm_oxide_b200.engine import Generator
    gen = Generator(llm_for(d, "float32", page))
    prompt = random_tokens(12, cfg.vocab_size, 77)
    full = gen.greedy(prompt, 10).tokens
    stop = full[3]
    cut = gen.greedy(prompt, 10, stop).tokens
    assert cut == full[:full.index(stop) + 1]           # crates/engine/src/generate.rs:176-184


def test_driver_errors(tmp_path_factory):
    from vllm_oxide_b200.engine import Generator
    from vllm_oxide_b200.errors import CapacityError, ShapeError
    cfg, _, page = TINY["A"]
    d = make_model_dir(tmp_path_factory.getbasetemp(), "A")
    gen = Generator(llm_for(d, "float32", page, max_model_len=32))
    with pytest.raises(ShapeError):                      # crates/engine/src/generate.rs:55-60
        gen.greedy([], 4)
    with pytest.raises(ShapeError):
        gen.greedy([1, 2], 0)
    with pytest.raises(CapacityError):                   # crates/engine/src/generate.rs:187-193
        gen.greedy(list(range(30)), 4)
    gen.greedy(list(range(30)), 3)                       # 30 + 3 - 1 = 32 fits exactly
    with pytest.raises(ShapeError, match="vocabulary"):
        gen.greedy([cfg.vocab_size], 2)


@pytest.mark.parametrize("name", ["B", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batched_equals_alone_and_graphs_change_nothing(tmp_path_factory, dtype, name):
    """Tokens of a request do not depend on what is scheduled beside it (CLAUDE.md:72), nor on
    whether its decode steps are replayed from CUDA graphs, in either dtype."""
    cfg, _, page = TINY[name]
    d = make_model_dir(tmp_path_factory.getbasetemp(), name)
    prompts = [random_tokens(L, cfg.vocab_size, 200 + i) for i, L in enumerate([1, 9, 40, 70, 23, 3])]
    params = [sp(max_new_tokens=12, temperature=0.0 if i % 2 == 0 else 0.7, seed=40 + i, stop_token_ids=()) for i in range(6)]
    alone = []
    solo = llm_for(d, dtype, page, cuda_graphs=False)
    for p, s in zip(prompts, params):
        alone.append(solo.generate([p], s)[0].token_ids)
    for graphs in (False, True):
        llm = llm_for(d, dtype, page, cuda_graphs=graphs, prefill_chunk=16, max_batch_tokens=40)
        outs = llm.generate(prompts, params)
        # float32: exact. bfloat16: steps of different sizes use different kernels (and so round
        # differently), so a pick may differ where the oracle's logits are tied within the tolerance.
        for p, prm, o, a in zip(prompts, params, outs, alone):
            assert_same_or_near_tie(d, p, o.token_ids, a, prm, 0.0 if dtype == "float32" else TOL[torch.bfloat16])
        assert all(o.finish_reason == "length" for o in outs)
        assert llm.stats["graph_steps"] > 0 if graphs else llm.stats["graph_steps"] == 0
        assert llm.runner.manager.check_invariants() == ""


def test_temperature_sampling_equals_plain_rule(tmp_path_factory):
    """Seeded temperature sampling (BASELINE tiny B: 0.7) picks what the plain Gumbel-max rule
    picks from the plain logits, as long as the pick is not a near-tie."""
    cfg, _, page = TINY["B"]
    d = make_model_dir(tmp_path_factory.getbasetemp(), "B")
    pc, pt = plain.load_model(d)
    llm = llm_for(d, "float32", page)
    prompt = random_tokens(9, cfg.vocab_size, 5)
    out = llm.generate([prompt], sp(max_new_tokens=6, temperature=0.7, seed=(3 << 32) | 12345, stop_token_ids=()))[0]
    seq = list(prompt)
    for i, tok in enumerate(out.token_ids):
        logits = plain.forward(pc, pt, seq)[-1]
        assert tok == plain.temperature_pick(logits.float(), 0.7, (3 << 32) | 12345, i)
        seq.append(tok)
    other = llm.generate([prompt], sp(max_new_tokens=6, temperature=0.7, seed=999, stop_token_ids=()))[0]
    assert other.token_ids != out.token_ids


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_preemption_recomputes_and_changes_no_token(tmp_path_factory, dtype):
    cfg, _, page = TINY["A"]
    d = make_model_dir(tmp_path_factory.getbasetemp(), "A")
    prompts = [random_tokens(L, cfg.vocab_size, 300 + i) for i, L in enumerate([30, 28, 25, 31])]
    params = sp(max_new_tokens=40, stop_token_ids=())
    roomy = llm_for(d, dtype, page, cuda_graphs=False).generate(prompts, params)
    # 12 pages of 16 = 192 tokens for four requests that grow to ~70 each: someone must give way
    tight = llm_for(d, dtype, page, num_pages=12, cuda_graphs=False)
    outs = tight.generate(prompts, params)
    assert tight.stats["preemptions"] > 0 and sum(o.preemptions for o in outs) == tight.stats["preemptions"]
    # float32: exact. bfloat16: recomputing a generated token as part of a prompt portion may round
    # differently, so a pick may differ where the oracle's logits are tied within the tolerance
    for p, o, r in zip(prompts, outs, roomy):
        assert_same_or_near_tie(d, p, o.token_ids, r.token_ids, params, 0.0 if dtype == "float32" else TOL[torch.bfloat16])
    assert tight.runner.manager.num_free_pages(0) == 12 and tight.runner.manager.check_invariants() == ""


def test_request_too_large_for_the_pool_fails_cleanly(tmp_path_factory):
    from vllm_oxide_b200.errors import CapacityError
    cfg, _, page = TINY["A"]
    d = make_model_dir(tmp_path_factory.getbasetemp(), "A")
    llm = llm_for(d, "float32", page, num_pages=2)
    with pytest.raises(CapacityError):
        llm.generate([list(range(40))], sp(max_new_tokens=4))
    out = llm.generate([list(range(20))], sp(max_new_tokens=4, stop_token_ids=()))[0]
    assert out.finish_reason == "length" and len(out.token_ids) == 4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_long_decoding_and_first_tokens(tmp_path_factory, dtype):
    """220 single-token steps from an empty cache (the first tokens of a sequence are steps like
    any other), each position compared with the plain implementation."""
    from tests.test_gpu_replay import _session, run_trace, check
    cfg, _, page = TINY["A"]
    d = make_model_dir(tmp_path_factory.getbasetemp(), "A")
    toks = random_tokens(220, cfg.vocab_size, 8)
    s = _session(d, dtype, 256, page)
    steps = [{"step": i, "entries": [{"id": "x", "tokens": [toks[i]], "want": [0]}], "end": ["x"] if i == 219 else []}
             for i in range(220)]
    got = run_trace(s, steps)
    assert len(got) == 220
    check(got, d, {"x": toks}, dtype, "token by token")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_workspace_formula_is_the_high_water_mark_of_the_largest_step(tmp_path_factory, name, dtype):
    """The step workspace is sized by a formula (the reference's arena formula,
    crates/engine/src/model.rs:68-90): after a step of as many tokens as the engine admits, wanting
    every row's logits, the workspace's high-water mark EQUALS the formula (the reference's own
    test, crates/engine/src/model.rs:400-419), and smaller steps stay below it."""
    from vllm_oxide_b200.config import EngineConfig
    from vllm_oxide_b200.engine import ModelRunner
    cfg, _, page = TINY[name]
    d = make_model_dir(tmp_path_factory.getbasetemp(), name)
    eng = EngineConfig(max_batch_tokens=96, max_seqs=4, max_model_len=96, block_size=page, num_pages=4 * 96 // page,
                       dtype=dtype, cuda_graphs=False)
    r = ModelRunner.from_dir(d, eng)
    toks = random_tokens(96, cfg.vocab_size, 3)
    r.admit(1)
    r.manager.reserve(1, 96)
    out = torch.empty((96, cfg.vocab_size), dtype=torch.float32)
    r.step(r.build_arrays([r.rt.StepEntry(1, toks, list(range(96)))]), logits_out=out)
    torch.cuda.synchronize()
    assert r.workspace.high_water == r.workspace_bytes == r.workspace_formula(r.rows_cap)
    r.workspace.high_water = 0
    for n in (1, 7, 33, 64):                               # other row counts take other paths through the parts
        r.admit(2)
        r.manager.reserve(2, n)
        r.step(r.build_arrays([r.rt.StepEntry(2, toks[:n], list(range(n)))]), logits_out=out)
        torch.cuda.synchronize()
        r.manager.release(2)
        assert r.workspace.high_water <= r.workspace_formula(n) <= r.workspace_bytes
    pc, pt = plain.load_model(d)
    assert max_rel_diff(out[-1], plain.forward(pc, pt, toks)[-1]) <= TOL[torch.float32 if dtype == "float32" else torch.bfloat16]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_running_ahead_changes_no_token_and_sees_stop_tokens(tmp_path_factory, dtype):
    """Steady decode steps are launched one ahead of the host's reads. Outputs are the same with
    and without, for requests that run to their length and for requests that meet a stop token
    (seen one step late: what was computed past it is dropped)."""
    cfg, _, page = TINY["B"]
    d = make_model_dir(tmp_path_factory.getbasetemp(), "B")
    prompts = [random_tokens(L, cfg.vocab_size, 700 + i) for i, L in enumerate([3, 11, 26, 7, 19])]
    free = sp(max_new_tokens=30, stop_token_ids=())
    base = llm_for(d, dtype, page, run_ahead=False)
    full = [o.token_ids for o in base.generate(prompts, free)]
    assert base.stats["ahead_steps"] == 0
    # stop tokens that come up at different places (a request's own 4th, 9th, ... token), one request without
    params = [sp(max_new_tokens=30, stop_token_ids=(full[i][3 + 5 * i],)) if i < 4 else free for i in range(5)]
    want = base.generate(prompts, params)
    assert [o.finish_reason for o in want][:4] == ["stop"] * 4 and want[4].finish_reason == "length"
    ahead = llm_for(d, dtype, page, run_ahead=True)
    got = ahead.generate(prompts, params)
    assert ahead.stats["ahead_steps"] > 0
    for g, w, p, prm in zip(got, want, prompts, params):
        assert g.finish_reason == w.finish_reason
        assert_same_or_near_tie(d, p, g.token_ids, w.token_ids, prm, 0.0 if dtype == "float32" else TOL[torch.bfloat16])
    for p, o, w in zip(prompts, ahead.generate(prompts, free), full):
        assert_same_or_near_tie(d, p, o.token_ids, w, free, 0.0 if dtype == "float32" else TOL[torch.bfloat16])
    assert ahead.runner.manager.check_invariants() == ""
    assert ahead.runner.manager.num_free_pages(0) == ahead.runner.manager.num_pages(0)


def test_generation_crosses_into_long_contexts(tmp_path_factory):
    """A request grows past the length from which decode steps count as long-context ones: the
    replayed graphs change kind on the way, and the tokens are those of steps launched one by one."""
    from vllm_oxide_b200.tuning import TUNING
    LONG_CONTEXT_KEYS = TUNING.long_context_keys
    cfg, _, page = TINY["DL"]
    d = make_model_dir(tmp_path_factory.getbasetemp(), "DL")
    prompts = [random_tokens(LONG_CONTEXT_KEYS - 6, cfg.vocab_size, 41), random_tokens(40, cfg.vocab_size, 42)]
    params = sp(max_new_tokens=16, stop_token_ids=())
    kw = dict(max_model_len=LONG_CONTEXT_KEYS + 64, max_batch_tokens=2048, num_pages=(LONG_CONTEXT_KEYS + 256) // page + 8)
    plain_steps = llm_for(d, "bfloat16", page, cuda_graphs=False, run_ahead=False, **kw)
    want = plain_steps.generate(prompts, params)
    graphs = llm_for(d, "bfloat16", page, cuda_graphs=True, run_ahead=True, **kw)
    got = graphs.generate(prompts, params)
    kinds = {key[2] for key in graphs.runner._graphs}
    assert kinds == {False, True}, kinds
    for g, w, p in zip(got, want, prompts):
        assert_same_or_near_tie(d, p, g.token_ids, w.token_ids, params, TOL[torch.bfloat16])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_replayed_from_graphs_give_the_same_tokens(tmp_path_factory, dtype):
    """Steps that are no decode steps (portions of prompts, mixed batches) are recorded as CUDA
    graphs when their shape class comes again, rows padded up to the class; the tokens are those of
    steps launched one by one."""
    name = "B" if dtype == "float32" else "D"
    cfg, _, page = TINY[name]
    d = make_model_dir(tmp_path_factory.getbasetemp(), name)
    # prompts of 130..150 tokens cut into portions of 48: every request brings portions of 48, 48
    # and a rest that falls into one class of rows
    prompts = [random_tokens(130 + 3 * i, cfg.vocab_size, 60 + i) for i in range(6)]
    params = sp(max_new_tokens=6, stop_token_ids=())
    kw = dict(max_batch_tokens=48, max_seqs=4, max_model_len=256, num_pages=4 * 256 // page)
    want = [o.token_ids for o in llm_for(d, dtype, page, step_graphs=0, **kw).generate(prompts, params)]
    llm = llm_for(d, dtype, page, step_graphs=2, **kw)
    got = [o.token_ids for o in llm.generate(prompts, params)]
    assert llm.runner.step_graph_replays > 4 and len(llm.runner._step_graphs) >= 1
    for g, w, p in zip(got, want, prompts):
        assert_same_or_near_tie(d, p, g, w, params, 0.0 if dtype == "float32" else TOL[torch.bfloat16])
    assert llm.runner.manager.num_free_pages(0) == llm.runner.manager.num_pages(0)


def test_tight_pool_and_replayed_steps_change_no_token_in_f32():
    """Forty requests of 5 to 700 tokens, greedy and with temperature, once with room for all and
    steps launched one by one, once with a pool so tight that requests are preempted and
    recomputed, a smaller token budget, and every step that is no decode step recorded as a CUDA
    graph at its first sighting: in float32 the tokens are the same to the last one, nothing leaks."""
    from vllm_oxide_b200 import models
    from vllm_oxide_b200.config import EngineConfig, LlamaConfig
    from vllm_oxide_b200.engine import LLM, ModelRunner
    from vllm_oxide_b200.weights import random_tensors
    cfg = LlamaConfig(hidden_size=192, intermediate_size=320, num_hidden_layers=3, num_attention_heads=6,
                      num_key_value_heads=2, head_dim=32, vocab_size=1000, max_position_embeddings=4096,
                      rms_norm_eps=1e-5, rope_theta=10000.0, rope_scaling=None, tie_word_embeddings=False)
    tensors = random_tensors(models.llama_manifest(cfg), 0, 0.08, torch.float32, "cuda:0")
    n = 40
    g = torch.Generator().manual_seed(3)
    lens = torch.randint(5, 700, (n,), generator=g).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (k,), generator=g).tolist() for k in lens]
    params = [sp(max_new_tokens=40 + i % 30, temperature=0.0 if i % 3 else 0.8, seed=i, stop_token_ids=()) for i in range(n)]
    outs = []
    for pages, graphs_after, budget in ((n * 64, 0, 512), (300, 1, 256)):
        eng = EngineConfig(max_batch_tokens=budget, max_seqs=16, max_model_len=1024, num_pages=pages, step_graphs=graphs_after,
                           dtype="float32")
        llm = LLM(ModelRunner(cfg, tensors, eng))
        outs.append([o.token_ids for o in llm.generate(prompts, params)])
        r = llm.runner
        assert r.manager.check_invariants() == "" and r.manager.num_free_pages(0) == r.manager.num_pages(0)
        if graphs_after:
            assert llm.stats["preemptions"] > 0 and r.step_graph_replays > 0
    assert outs[0] == outs[1]


@pytest.mark.parametrize("seed", range(12))
def test_random_models_and_engine_settings_change_no_token_in_f32(seed):
    """Drawn from the seed: a small model (head size 16 to 128, heads and groups, widths that are no
    power of two, tied or own output head, llama3 scaling or none), a handful of requests with greedy
    and temperature sampling and stop tokens, and engine settings (page size, token budget, requests
    per step, a pool from just enough for one request to most of what all need, graphs of either kind
    on or off, running ahead or not). In float32 the tokens equal those of a roomy engine that
    launches step by step, and no page is lost."""
    import random
    from vllm_oxide_b200 import models
    from vllm_oxide_b200.config import EngineConfig, LlamaConfig, RopeScaling
    from vllm_oxide_b200.engine import LLM, ModelRunner
    from vllm_oxide_b200.weights import random_tensors
    rnd = random.Random(1000 + seed)
    hd, kv, group = rnd.choice([16, 32, 64, 128]), rnd.choice([1, 2, 4]), rnd.choice([1, 2, 4])
    vocab = rnd.choice([500, 1000, 1531])
    cfg = LlamaConfig(hidden_size=rnd.choice([96, 160, 192, 256]), intermediate_size=rnd.choice([200, 320, 512]),
                      num_hidden_layers=rnd.choice([1, 2, 3]), num_attention_heads=kv * group, num_key_value_heads=kv, head_dim=hd,
                      vocab_size=vocab, max_position_embeddings=4096, rms_norm_eps=1e-5, rope_theta=10000.0,
                      rope_scaling=rnd.choice([None, RopeScaling(8.0, 1.0, 4.0, 64)]), tie_word_embeddings=rnd.choice([True, False]))
    tensors = random_tensors(models.llama_manifest(cfg), seed, 0.08, torch.float32, "cuda:0")
    n = rnd.randint(6, 24)
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(2, rnd.choice([60, 300]), (n,), generator=g).tolist()
    prompts = [torch.randint(0, vocab, (k,), generator=g).tolist() for k in lens]
    params = [sp(max_new_tokens=rnd.randint(1, 40), temperature=0.0 if rnd.random() < 0.6 else 0.8, seed=i,
                 stop_token_ids=rnd.choice([(), (3, 7, 11)])) for i in range(n)]
    page = rnd.choice([8, 16, 32])
    longest = max(k + p.max_new_tokens for k, p in zip(lens, params))
    max_len = -(-longest // page) * page + page
    per_request = max_len // page
    roomy = dict(max_batch_tokens=1024, max_seqs=n, num_pages=n * per_request + 8, step_graphs=0, cuda_graphs=False, run_ahead=False)
    drawn = dict(max_batch_tokens=rnd.choice([16, 64, 256]), max_seqs=rnd.choice([2, 4, 8, 16]),
                 num_pages=max(per_request + 1, int(rnd.uniform(0.15, 0.7) * n * per_request)),
                 step_graphs=rnd.choice([0, 1, 2]), cuda_graphs=rnd.choice([True, False]), run_ahead=rnd.choice([True, False]))
    outs = []
    for kw in (roomy, drawn):
        llm = LLM(ModelRunner(cfg, tensors, EngineConfig(max_model_len=max_len, block_size=page, dtype="float32", **kw)))
        outs.append([o.token_ids for o in llm.generate(prompts, params)])
        r = llm.runner
        assert r.manager.check_invariants() == "" and r.manager.num_free_pages(0) == r.manager.num_pages(0), kw
    assert outs[0] == outs[1], drawn
    assert all(1 <= len(t) <= p.max_new_tokens for t, p in zip(outs[0], params))


@pytest.mark.parametrize("run_ahead", [False, True])
def test_tokens_are_reported_as_they_are_read(tmp_path_factory, run_ahead):
    """`on_token`: every generated token once, in order, the stop token included, nothing that was
    computed past a stop token; with and without steps launched ahead."""
    cfg, _, page = TINY["B"]
    d = make_model_dir(tmp_path_factory.getbasetemp(), "B")
    prompts = [random_tokens(L, cfg.vocab_size, 800 + i) for i, L in enumerate([4, 13, 30, 9])]
    base = llm_for(d, "float32", page, run_ahead=False)
    full = [o.token_ids for o in base.generate(prompts, sp(max_new_tokens=24, stop_token_ids=()))]
    params = [sp(max_new_tokens=24, stop_token_ids=(full[i][5 + 4 * i],)) if i < 3 else sp(max_new_tokens=24, stop_token_ids=())
              for i in range(4)]
    llm = llm_for(d, "float32", page, run_ahead=run_ahead)
    seen = {i: [] for i in range(4)}
    outs = llm.generate(prompts, params, on_token=lambda i, tok: seen[i].append(tok))
    assert [o.finish_reason for o in outs] == ["stop", "stop", "stop", "length"]
    assert [seen[i] for i in range(4)] == [o.token_ids for o in outs]
    assert llm.on_token is None
    assert (llm.stats["ahead_steps"] > 0) == run_ahead


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_more_state_slots_than_a_step_has_rows(tmp_path_factory, dtype):
    """max_seqs above max_batch_tokens (a natural configuration for tests): a decode step then holds
    at most max_batch_tokens requests, and the graphs' batch classes stop there."""
    name = "A" if dtype == "float32" else "D"
    cfg, _, page = TINY[name]
    d = make_model_dir(tmp_path_factory.getbasetemp(), name)
    prompts = [random_tokens(3 + i % 5, cfg.vocab_size, 900 + i) for i in range(30)]
    params = sp(max_new_tokens=40, stop_token_ids=())       # long enough for all 30 to be decoding at once
    kw = dict(max_batch_tokens=24, max_seqs=32, max_model_len=64, num_pages=32 * 64 // page)
    want = [o.token_ids for o in llm_for(d, dtype, page, cuda_graphs=False, **kw).generate(prompts, params)]
    llm = llm_for(d, dtype, page, cuda_graphs=True, **kw)
    got = [o.token_ids for o in llm.generate(prompts, params)]
    assert llm.runner.decode_cap == 24 and max(key[0] for key in llm.runner._graphs) == 24
    for p, g, w in zip(prompts, got, want):
        assert_same_or_near_tie(d, p, g, w, params, 0.0 if dtype == "float32" else TOL[torch.bfloat16])
    assert llm.runner.manager.num_free_pages(0) == llm.runner.manager.num_pages(0)
