"""The scheduler's decisions (no GPU): budget, chunking, decode first, admission, preemption,
finishing and freeing, and what happens when pages run out."""
import random

import pytest

from vllm_oxide_b200.csrc.build import runtime_module

rt = runtime_module()


def make(pages=64, page=4, slots=8, budget=16, max_seqs=8, max_len=256, chunk=0):
    c = rt.CacheManager(page, [rt.GroupSpec(rt.FULL, 0, pages)], slots)
    return c, rt.Scheduler(c, budget, max_seqs, max_len, chunk)


def sp(n=4, stop=(), temp=0.0, seed=0):
    return rt.SamplingParams(n, temp, seed, list(stop))


def run_step(s, token=lambda rid, k: 100 + k):
    plan = s.schedule()
    sampled = [token(e.id, i) for i, e in enumerate(plan.entries) if e.sample]
    return plan, s.update(plan, sampled)


def test_prompt_is_cut_into_portions_under_the_budget():
    c, s = make(budget=16)
    s.add_request(1, list(range(40)), sp(3))
    plan, done = run_step(s)
    assert [(e.id, e.start, e.count, e.sample) for e in plan.entries] == [(1, 0, 16, False)] and plan.admitted == [1]
    plan, _ = run_step(s)
    assert [(e.start, e.count, e.sample) for e in plan.entries] == [(16, 16, False)]
    plan, _ = run_step(s)
    assert [(e.start, e.count, e.sample) for e in plan.entries] == [(32, 8, True)]      # reaches the end: a token is picked
    plan, _ = run_step(s)
    assert [(e.start, e.count, e.sample) for e in plan.entries] == [(40, 1, True)]       # decoding
    plan, done = run_step(s)
    assert [f.reason for f in done] == ["length"] and len(done[0].output) == 3
    assert not s.has_unfinished() and c.num_free_pages(0) == 64 and c.num_free_slots() == 8


def test_decodes_go_first_and_share_the_step_with_a_portion():
    c, s = make(budget=16, chunk=8)
    s.add_request(1, [1, 2, 3], sp(10))
    run_step(s)                                   # request 1 prefilled, now decoding
    s.add_request(2, list(range(30)), sp(2))
    plan, _ = run_step(s)
    assert [(e.id, e.count) for e in plan.entries] == [(1, 1), (2, 8)]      # decode first, then a portion of 8 (prefill_chunk)
    plan, _ = run_step(s)
    assert [(e.id, e.start, e.count) for e in plan.entries] == [(1, 4, 1), (2, 8, 8)]
    total = sum(e.count for e in plan.entries)
    assert total <= 16


def test_budget_and_sequence_limits_hold():
    c, s = make(budget=10, max_seqs=3, pages=256)
    for i in range(6):
        s.add_request(i, list(range(7)), sp(5))
    seen_running = 0
    for _ in range(60):
        if not s.has_unfinished():
            break
        plan, _ = run_step(s)
        assert sum(e.count for e in plan.entries) <= 10 and len(plan.entries) <= 3
        seen_running = max(seen_running, s.num_running())
        assert c.check_invariants() == ""
    assert not s.has_unfinished() and seen_running == 3


def test_stop_token_is_kept_and_frees_at_once():
    c, s = make()
    s.add_request(1, [5, 6], sp(10, stop=(77,)))
    run_step(s, token=lambda rid, k: 9)
    plan, done = run_step(s, token=lambda rid, k: 77)
    assert [f.reason for f in done] == ["stop"] and done[0].output == [9, 77]       # crates/engine/src/generate.rs:105-108
    assert c.num_requests() == 0


def test_capacity_rule_of_the_reference():
    # prompt + max_new - 1 must fit the model length and the pool (crates/engine/src/generate.rs:64-71)
    c, s = make(max_len=10, pages=64)
    s.add_request(1, list(range(8)), sp(3))                 # 8 + 3 - 1 = 10: fits
    with pytest.raises(rt.RuntimeFault, match="capacity"):
        s.add_request(2, list(range(8)), sp(4))             # 11 > 10
    with pytest.raises(rt.RuntimeFault, match="empty prompt or max_new = 0"):
        s.add_request(3, [], sp(1))
    c2, s2 = make(pages=2, page=4, max_len=100)
    with pytest.raises(rt.RuntimeFault, match="pages"):
        s2.add_request(1, list(range(9)), sp(1))            # 3 pages needed, the pool has 2


def test_out_of_pages_preempts_the_latest_and_recomputes_it():
    # 6 pages of 4 tokens; two requests that together outgrow the pool while decoding
    c, s = make(pages=6, page=4, budget=64, max_len=64)
    s.add_request(1, list(range(8)), sp(12))
    s.add_request(2, list(range(8)), sp(12))
    preempted_at = None
    outputs = {}
    for step in range(80):
        if not s.has_unfinished():
            break
        plan, done = run_step(s, token=lambda rid, k: 50 + rid)
        if plan.preempted and preempted_at is None:
            preempted_at = step
            assert plan.preempted == [2]                    # the most recently admitted one
            assert s.waiting() == [2] and s.running() == [1]
            assert s.computed_of(2) == 0 and s.preemptions_of(2) == 1
            assert not any(e.id == 2 for e in plan.entries) and not plan.admitted
        for f in done:
            outputs[f.id] = (f.reason, f.output)
        assert c.check_invariants() == ""
    assert preempted_at is not None
    assert outputs[1] == ("length", [51] * 12) and outputs[2] == ("length", [52] * 12)
    assert c.num_free_pages(0) == 6
    # after preemption request 2 is prefilled again over prompt + what it had generated


def test_recompute_covers_prompt_plus_generated():
    c, s = make(pages=6, page=4, budget=64, max_len=64)
    s.add_request(1, list(range(8)), sp(12))
    s.add_request(2, list(range(8)), sp(12))
    readmitted = None
    for _ in range(80):
        if not s.has_unfinished():
            break
        plan, _ = run_step(s)
        if 2 in plan.admitted and s.preemptions_of(2) == 1 and readmitted is None:
            e = [e for e in plan.entries if e.id == 2][0]
            readmitted = (e.start, e.count, len(s.tokens_of(2)) - (1 if e.sample else 0))
    # it starts again at token 0 and has more than its 8-token prompt to work through
    assert readmitted is not None and readmitted[0] == 0 and readmitted[2] > 8


def test_alone_and_out_of_pages_is_a_capacity_finish():
    # a window-free pool too small for the request's growth cannot be entered at all (add_request
    # refuses); a request that shrank the pool for itself is the only other way: simulate by
    # holding pages outside the scheduler
    c, s = make(pages=4, page=4, budget=64, max_len=64)
    c.admit(999)
    c.reserve(999, 8)                                       # someone else holds 2 of the 4 pages
    s.add_request(1, list(range(6)), sp(8))                 # needs 4 pages in the end
    reasons = []
    for _ in range(40):
        if not s.has_unfinished():
            break
        plan, done = run_step(s)
        reasons += [(f.id, f.reason, len(f.output)) for f in done]
    assert reasons == [(1, "capacity", 3)]                  # 8 tokens fit: 6 prompt + 2 fed back; the third pick has no page to go to
    assert c.num_free_pages(0) == 2 and c.check_invariants() == ""


def test_a_portion_shrinks_to_the_pages_that_are_left():
    c, s = make(pages=8, page=4, budget=64, max_len=64)
    s.add_request(1, list(range(4)), sp(9))
    run_step(s)
    s.add_request(2, list(range(30)), sp(1))                # fits the pool alone (8 pages), not beside request 1
    with pytest.raises(rt.RuntimeFault):
        s.add_request(3, list(range(40)), sp(1))            # can never fit: refused at once
    plan, _ = run_step(s)
    # request 1 decodes (its second page); request 2 gets what is left (6 pages -> 24 tokens), nobody is preempted
    assert [(e.id, e.count) for e in plan.entries] == [(1, 1), (2, 24)] and not plan.preempted


def test_abort():
    c, s = make()
    s.add_request(1, [1, 2, 3], sp(5))
    run_step(s)
    assert s.abort(1) and not s.abort(1)
    assert [f.reason for f in s.take_done()] == ["abort"]
    assert c.num_requests() == 0 and not s.has_unfinished()


@pytest.mark.parametrize("seed", range(5))
def test_random_traces_finish_everything_and_leak_nothing(seed):
    rng = random.Random(seed)
    pages, page = 24, 4
    c, s = make(pages=pages, page=page, slots=5, budget=rng.choice([8, 16, 33]), max_seqs=5, max_len=96,
                chunk=rng.choice([0, 3, 7]))
    want, got, next_id = {}, {}, 0
    for step in range(3000):
        if next_id < 25 and rng.random() < 0.3:
            p = rng.randrange(1, 40)
            n = rng.randrange(1, 20)
            try:
                s.add_request(next_id, [rng.randrange(50) for _ in range(p)], sp(n))
                want[next_id] = n
            except rt.RuntimeFault:
                pass
            next_id += 1
        if not s.has_unfinished():
            if next_id >= 25:
                break
            continue
        plan, done = run_step(s, token=lambda rid, k: rid)
        ids = [e.id for e in plan.entries]
        assert len(ids) == len(set(ids))
        assert sum(e.count for e in plan.entries) <= 33
        for f in done:
            got[f.id] = f
        assert c.check_invariants() == "", c.check_invariants()
    assert not s.has_unfinished()
    assert set(got) == set(want)
    for rid, f in got.items():
        assert f.reason == "length" and f.output == [rid] * want[rid]      # preempted or not, the output is whole
    assert c.num_free_pages(0) == pages and c.num_free_slots() == 5


# ----------------------------------------------------------------------------- running ahead of the host's reads
def _ahead_run(s, tokens_of, stops_seen=None):
    """Drive the scheduler the way the engine does when it launches step n + 1 before it reads
    step n. `tokens_of(id, k)` is the k-th generated token of a request. Returns what ended."""
    count, ended, flight = {}, [], None

    def picks(plan):
        out = []
        for e in plan.entries:
            k = count.get(e.id, 0)
            out.append(tokens_of(e.id, k))
            count[e.id] = k + 1
        return out
    guard = 0
    while s.has_unfinished() or flight is not None:
        guard += 1
        assert guard < 500
        if flight is None:
            if s.steady_decode():
                plan = s.schedule()
                assert plan.decode_only and not plan.preempted and not plan.admitted
                toks = picks(plan)
                s.advance(plan)
                flight = (plan, toks, list(s.running()))
            else:
                plan = s.schedule()
                ended += s.update(plan, [tokens_of(e.id, count.setdefault(e.id, 0)) for e in plan.entries if e.sample])
                for e in plan.entries:
                    if e.sample:
                        count[e.id] += 1
            continue
        nxt = None
        if s.steady_decode() and list(s.running()) == flight[2]:
            plan = s.schedule()
            assert [e.id for e in plan.entries] == flight[2]
            toks = picks(plan)
            s.advance(plan)
            nxt = (plan, toks, list(s.running()))
        got = s.resolve(flight[0], flight[1], 1 if nxt else 0)
        ended += got
        if got and nxt:
            ended += s.resolve(nxt[0], nxt[1], 0)
            nxt = None
        flight = nxt
    return ended


@pytest.mark.parametrize("seed", [0, 1, 2, 3])
def test_running_ahead_gives_the_same_outputs_as_reading_every_step(seed):
    """Requests of different lengths, some with stop tokens that come up mid-way, through the
    run-ahead protocol and through plain update(): same outputs, same reasons, nothing leaks."""
    rng = random.Random(seed)
    reqs = []
    for i in range(6):
        prompt = [rng.randrange(50) for _ in range(rng.randrange(1, 12))]
        n = rng.randrange(1, 14)
        stop = [7] if i % 2 == 0 else []
        reqs.append((i, prompt, n, stop))
    gen = {i: [rng.choice([3, 5, 7, 9, 11]) for _ in range(20)] for i, *_ in reqs}
    tokens_of = lambda rid, k: gen[rid][k]

    c1, s1 = make(pages=64, page=4, budget=16)
    c2, s2 = make(pages=64, page=4, budget=16)
    for i, prompt, n, stop in reqs:
        s1.add_request(i, prompt, sp(n, stop))
        s2.add_request(i, prompt, sp(n, stop))
    plain_done, count = [], {}
    while s1.has_unfinished():
        plan = s1.schedule()
        sampled = []
        for e in plan.entries:
            if e.sample:
                sampled.append(tokens_of(e.id, count.get(e.id, 0)))
                count[e.id] = count.get(e.id, 0) + 1
        plain_done += s1.update(plan, sampled)
    ahead_done = _ahead_run(s2, tokens_of)
    key = lambda fs: sorted((f.id, f.reason, tuple(f.output)) for f in fs)
    assert key(ahead_done) == key(plain_done)
    assert c2.check_invariants() == "" and c2.num_free_pages(0) == 64 and c2.num_free_slots() == 8


def test_steady_decode_is_false_whenever_the_next_step_could_differ():
    c, s = make(pages=8, page=4, budget=16)
    s.add_request(1, [1, 2, 3], sp(4))
    assert not s.steady_decode()                     # still waiting
    run_step(s)
    assert s.steady_decode()                         # decoding, 1 of 4 generated
    s.add_request(2, [4, 5], sp(4))
    assert not s.steady_decode()                     # someone waits
    run_step(s)
    assert s.steady_decode()
    run_step(s)                                      # request 1 has 3 of 4: its next token ends it by length
    assert not s.steady_decode()
    c2, s2 = make(pages=3, page=4, budget=16)
    s2.add_request(1, list(range(7)), sp(6))
    s2.add_request(2, [1], sp(6))
    run_step(s2)
    assert c2.num_free_pages(0) == 0 and not s2.steady_decode()      # no free page for every running request


def test_admission_watermark_keeps_room_for_the_running_requests():
    """With a watermark a waiting request is admitted only if so many pages stay free behind its
    first portion while others run; alone it is admitted anyway; 0 admits whenever a token fits."""
    c, s = make(pages=8, page=4, budget=64, max_len=64)
    s.set_admission_watermark(3)
    assert s.admission_watermark() == 3
    s.add_request(1, list(range(8)), sp(20))        # 2 pages
    s.add_request(2, list(range(12)), sp(4))        # 3 pages: 8 - 2 - 3 = 3 would stay free: admitted
    s.add_request(3, list(range(4)), sp(4))         # 1 page: 3 - 1 = 2 < 3: waits
    plan, _ = run_step(s)
    assert plan.admitted == [1, 2] and s.waiting() == [3]
    assert c.check_invariants() == ""
    # request 3 comes in once request 2 has finished and given its pages back
    admitted_at = None
    for step in range(40):
        plan, done = run_step(s)
        if 3 in plan.admitted:
            admitted_at = step
            assert 2 not in s.running()
            break
    assert admitted_at is not None
    while s.has_unfinished():
        run_step(s)
    assert c.num_free_pages(0) == 8 and c.check_invariants() == ""
    # nothing runs: the watermark does not hold a request back
    c2, s2 = make(pages=4, page=4, budget=64, max_len=64)
    s2.set_admission_watermark(3)
    s2.add_request(7, list(range(10)), sp(2))       # 3 pages of 4: only 1 would stay free
    plan, _ = run_step(s2)
    assert plan.admitted == [7]
    with pytest.raises(rt.RuntimeFault):
        s2.set_admission_watermark(-1)


@pytest.mark.parametrize("seed", range(4))
def test_random_traces_with_a_watermark_finish_everything_with_fewer_preemptions(seed):
    def run(watermark):
        rng = random.Random(seed)
        c, s = make(pages=24, page=4, slots=5, budget=16, max_seqs=5, max_len=96)
        s.set_admission_watermark(watermark)
        want, got, preempted = {}, {}, 0
        for rid in range(20):
            n = rng.randrange(4, 20)
            s.add_request(rid, [rng.randrange(50) for _ in range(rng.randrange(1, 40))], sp(n))
            want[rid] = n
        for step in range(4000):
            if not s.has_unfinished():
                break
            plan, done = run_step(s, token=lambda rid, k: rid)
            preempted += len(plan.preempted)
            for f in done:
                got[f.id] = f
            assert c.check_invariants() == ""
        assert not s.has_unfinished() and c.num_free_pages(0) == 24
        assert {i: len(f.output) for i, f in got.items()} == want
        assert all(f.output == [i] * want[i] for i, f in got.items())
        return preempted
    without, with_room = run(0), run(4)
    assert with_room <= without
