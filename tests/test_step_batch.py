"""The arrays of a step (no GPU), against the reference's own metadata example."""
import numpy as np
import pytest

from vllm_oxide_b200.csrc.build import runtime_module

rt = runtime_module()


def sec(a, key, n, g=None):
    L = a.layout
    o = L[key] if g is None else L[key][g]
    return a.data()[o:o + n].tolist()


def test_two_portions_flatten_like_the_reference():
    # crates/engine/src/backend/paged.rs:231-261: two sequences, (context 0, 5 new) and
    # (context 6, 3 new), block size 4 -> positions [0,1,2,3,4,6,7,8], row_num_keys = pos + 1,
    # last rows [4, 7]; slots follow each request's own table.
    c = rt.CacheManager(4, [rt.GroupSpec(rt.FULL, 0, 16)], 4)
    c.admit(1), c.admit(2)
    c.reserve(2, 6), c.commit(2, 6)
    c.reserve(1, 5), c.reserve(2, 3)
    e1 = rt.StepEntry(1, [10, 11, 12, 13, 14], [4])
    e2 = rt.StepEntry(2, [20, 21, 22], [2], 0.7, (5 << 32) | 9, 3)
    a = rt.build_step(c, [e1, e2], 16, 4, 16, 8, 100)
    assert (a.rows, a.seqs, a.logit_count, a.max_new, a.max_seq_len, a.any_sampling) == (8, 2, 2, 5, 9, True)
    assert sec(a, "tokens", 8) == [10, 11, 12, 13, 14, 20, 21, 22]
    assert sec(a, "positions", 8) == [0, 1, 2, 3, 4, 6, 7, 8]
    assert sec(a, "row_seq", 8) == [0, 0, 0, 0, 0, 1, 1, 1]
    assert sec(a, "seq_starts", 3) == [0, 5, 8]
    assert sec(a, "context_lens", 2) == [0, 6] and sec(a, "seq_lens", 2) == [5, 9]
    assert sec(a, "logit_rows", 2) == [4, 7]
    t1, t2 = c.block_table(1, 0), c.block_table(2, 0)
    want = [t1[p // 4] * 4 + p % 4 for p in range(5)] + [t2[p // 4] * 4 + p % 4 for p in (6, 7, 8)]
    assert sec(a, "slot_mapping", 8, 0) == want
    bt = np.array(sec(a, "block_tables", 4 * 8, 0)).reshape(4, 8)
    assert bt[0, :2].tolist() == t1 and bt[1, :3].tolist() == t2 and (bt[0, 2:] == -1).all()
    assert sec(a, "state_slots", 2) == [c.state_slot(1), c.state_slot(2)]
    # padding rows attend to nothing and write nothing
    assert sec(a, "positions", 16)[8:] == [-1] * 8 and sec(a, "slot_mapping", 16, 0)[8:] == [-1] * 8
    temps = np.array(sec(a, "temperature", 2), dtype=np.int32).view(np.float32)
    assert temps[0] == 0.0 and abs(temps[1] - 0.7) < 1e-7
    assert sec(a, "seeds", 4) == [0, 0, 9, 5] and sec(a, "sample_steps", 2) == [0, 3]


def test_leading_single_tokens_are_counted():
    """`lead_single`: how many requests at the front of the batch bring exactly one token (a
    mixed step hands their rows to the decode attention kernel); one behind a portion does not count."""
    c = rt.CacheManager(4, [rt.GroupSpec(rt.FULL, 0, 32)], 8)
    for r in (1, 2, 3, 4):
        c.admit(r)
    for r in (1, 2, 4):
        c.reserve(r, 5), c.commit(r, 5)
    for r, n in ((1, 1), (2, 1), (3, 6), (4, 1)):
        c.reserve(r, n)
    e = [rt.StepEntry(1, [7], [0]), rt.StepEntry(2, [8], [0]), rt.StepEntry(3, [1, 2, 3, 4, 5, 6], [5]), rt.StepEntry(4, [9], [0])]
    assert rt.build_step(c, e, 16, 8, 16, 8, 100).lead_single == 2
    assert rt.build_step(c, e[2:], 16, 8, 16, 8, 100).lead_single == 0
    assert rt.build_step(c, [e[0], e[1], e[3]], 16, 8, 16, 8, 100).lead_single == 3


def test_refusals():
    c = rt.CacheManager(4, [rt.GroupSpec(rt.FULL, 0, 8)], 4)
    c.admit(1)
    with pytest.raises(rt.RuntimeFault, match="holds pages for 0 tokens"):
        rt.build_step(c, [rt.StepEntry(1, [1, 2])], 16, 4, 16, 8, 100)
    c.reserve(1, 2)
    with pytest.raises(rt.RuntimeFault, match="outside the vocabulary"):
        rt.build_step(c, [rt.StepEntry(1, [1, 100])], 16, 4, 16, 8, 100)
    with pytest.raises(rt.RuntimeFault, match="wanted place"):
        rt.build_step(c, [rt.StepEntry(1, [1, 2], [2])], 16, 4, 16, 8, 100)
    with pytest.raises(rt.RuntimeFault, match="exceed the limit of 1"):
        rt.build_step(c, [rt.StepEntry(1, [1, 2])], 1, 4, 16, 8, 100)
    with pytest.raises(rt.RuntimeFault, match="appears twice"):
        rt.build_step(c, [rt.StepEntry(1, [1]), rt.StepEntry(1, [2])], 16, 4, 16, 8, 100)
    with pytest.raises(rt.RuntimeFault, match="brings no tokens"):
        rt.build_step(c, [rt.StepEntry(1, [])], 16, 4, 16, 8, 100)
    with pytest.raises(rt.RuntimeFault, match="not admitted"):
        rt.build_step(c, [rt.StepEntry(9, [1])], 16, 4, 16, 8, 100)


def test_layout_is_a_function_of_the_capacities():
    a = rt.step_layout(16, 4, 16, 2, 8)
    b = rt.step_layout(16, 4, 16, 2, 8)
    assert a == b and a["total"] % 4 == 0
    offs = [a["tokens"], a["positions"], a["row_seq"], a["seq_starts"], a["context_lens"], a["seq_lens"],
            a["state_slots"], a["logit_rows"], a["temperature"], a["seeds"], a["sample_steps"]] + a["slot_mapping"] + a["block_tables"]
    assert len(set(offs)) == len(offs) and all(o % 4 == 0 and o < a["total"] for o in offs)


def test_shape_class_of_a_step():
    """What a recorded step is replayed for: rows are padded up, the longest portion is an upper
    bound, requests / wanted rows / leading single tokens are exact; decode steps have their own graphs."""
    from vllm_oxide_b200.engine.runner import step_shape_class
    from vllm_oxide_b200.tuning import TUNING
    LONG_CONTEXT_KEYS = TUNING.long_context_keys
    assert step_shape_class(8, 8, 8, 1, 8, 300, 2048) is None                 # a decode step
    assert step_shape_class(100, 2, 0, 60, 0, 300, 2048) is None              # no logits wanted
    assert step_shape_class(1, 1, 1, 1, 1, 5, 2048) is None
    assert step_shape_class(9, 2, 2, 8, 1, 40, 2048) == (16, 2, 2, 16, 1, False)
    assert step_shape_class(33, 3, 3, 20, 2, 40, 2048) == (64, 3, 3, 64, 2, False)
    assert step_shape_class(2048, 1, 1, 2048, 0, 2048, 2048) == (2048, 1, 1, 2048, 0, False)
    assert step_shape_class(1999, 5, 4, 1930, 3, LONG_CONTEXT_KEYS + 1, 2048) == (2048, 5, 4, 1984, 3, True)
    assert step_shape_class(130, 2, 2, 129, 0, 500, 192) == (192, 2, 2, 192, 0, False)    # never beyond the engine's rows
    assert step_shape_class(40, 4, 4, 37, 0, 90, 48) == (48, 4, 4, 48, 0, False)


def test_how_decode_attention_shares_a_request_over_blocks():
    """The rule that picks blocks per request and kv head and the way they merge: whatever the counts,
    it names something the kernel takes (a cluster of at most 8, or with the merge through global
    memory at most 64 blocks), and the measured cases keep their choices."""
    from vllm_oxide_b200.parts.attention import decode_split_rule
    for sms in (1, 7, 108, 132, 148, 200):
        for kv in (1, 2, 3, 8, 16):
            for seqs in (1, 2, 3, 8, 17, 64, 500):
                for long_context in (False, True):
                    splits, wide = decode_split_rule(seqs, kv, sms, long_context)
                    assert 1 <= splits <= (64 if wide else 8) and (long_context or not wide)
    assert decode_split_rule(8, 8, 148, False) == (6, False)          # the benchmark's decode step
    assert decode_split_rule(64, 8, 148, False) == (1, False)
    assert decode_split_rule(1, 8, 148, True) == (55, True)           # one long request
    assert decode_split_rule(8, 8, 148, True) == (6, True)


def test_batch_size_classes_of_decode_steps():
    from vllm_oxide_b200.engine.runner import decode_bucket
    assert [decode_bucket(n) for n in range(1, 18)] == [1, 2, 3, 4, 6, 6, 8, 8, 12, 12, 12, 12, 16, 16, 16, 16, 24]
    assert [decode_bucket(n) for n in (24, 25, 32, 33, 48, 49, 64, 65, 96, 97, 150)] == [24, 32, 32, 48, 48, 64, 64, 96, 96, 128, 192]
    assert all(decode_bucket(n) >= n for n in range(1, 2000))
