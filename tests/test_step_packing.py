"""The packed integer buffer of a step: the general packer and the one for decoding steps agree, padding entries
are empty, and the block-table updates name what the device lacks (host side; no GPU needed)."""
import types

import numpy as np
import pytest

from vllm_cpp_b200.engine.step import MetaLayout, ModelRunner, StepEntry


def fake_runner(groups=1, page_size=16, num_slots=8, max_blocks=64):
    r = types.SimpleNamespace(page_size=page_size, page_sizes=[page_size] * groups, num_slots=num_slots,
                              max_blocks=[max_blocks] * groups, tables=[None] * groups,
                              _uploaded=[[0] * num_slots for _ in range(groups)], vocab_size=1000, max_positions=page_size * max_blocks)
    for name in ("_fill", "_fill_decode", "_table_updates", "_validate"):
        setattr(r, name, types.MethodType(getattr(ModelRunner, name), r))
    r.USER_INTS_PER_ENTRY = ModelRunner.USER_INTS_PER_ENTRY
    return r


def table(rng, blocks):
    return [int(p) for p in rng.permutation(500)[:blocks]]


@pytest.mark.parametrize("groups", [1, 2])
def test_the_two_packers_agree_on_decoding_steps(groups):
    rng = np.random.default_rng(groups)
    r = fake_runner(groups)
    entries = []
    for slot, pos in ((3, 0), (0, 15), (5, 16), (1, 700)):
        entries.append(StepEntry(slot, pos, [int(rng.integers(0, 1000))], [table(rng, pos // 16 + 1) for _ in range(groups)], [0]))
        for g in range(groups):
            r._uploaded[g][slot] = -(-pos // 16)      # what earlier steps of the request sent: the blocks of its tokens so far
    updates = r._table_updates(entries)
    assert [len(u[0]) for u in updates] == [2] * groups   # positions 0 and 16 open a block; 15 and 700 sit in blocks the device has
    bucket = 8
    lay = MetaLayout(bucket, bucket, bucket, bucket, groups, bucket * r.USER_INTS_PER_ENTRY)
    user = list(range(100, 132))
    fast, facts_fast = r._fill_decode(lay, entries, updates, user)
    slow, facts_slow = r._fill(lay, entries, updates)
    o = lay.offsets
    slow[o["user"][0]:o["user"][0] + len(user)] = user
    assert fast.dtype == slow.dtype == np.int32 and fast.shape == slow.shape == (lay.size,)
    assert np.array_equal(fast, slow)
    for key in ("host_q_len", "host_q_start", "host_ctx_len", "host_slots"):
        assert list(facts_fast[key]) == list(facts_slow[key])
    # padding entries: no tokens, no context, stored nowhere
    assert fast[o["q_len"][0] + 4:o["q_len"][1]].tolist() == [0] * 4 and fast[o["ctx_len"][0] + 4:o["ctx_len"][1]].tolist() == [0] * 4
    assert fast[o["slot_map0"][0] + 4:o["slot_map0"][1]].tolist() == [-1] * 4


def test_block_table_updates_name_what_the_device_lacks():
    rng = np.random.default_rng(0)
    r = fake_runner()
    t = table(rng, 10)
    first = StepEntry(2, 0, list(range(40)), [t], [39])               # positions 0..39: blocks 0, 1, 2
    idx, val = r._table_updates([first])[0]
    assert idx == [2 * 64 + b for b in range(3)] and val == t[:3]
    again = StepEntry(2, 40, list(range(8)), [t], [7])                # 40..47: still block 2
    assert r._table_updates([again])[0] == ([], [])
    more = StepEntry(2, 48, [1], [t], [0])                            # 48: block 3
    assert r._table_updates([more])[0] == ([2 * 64 + 3], [t[3]])
    restart = StepEntry(2, 0, [1, 2], [t], [1])                       # the slot starts again from nothing
    assert r._table_updates([restart])[0] == ([2 * 64], [t[0]])
    short = StepEntry(4, 0, list(range(40)), [t[:2]], [39])
    with pytest.raises(ValueError, match="does not reach"):
        r._table_updates([short])


def test_a_portion_is_packed_with_positions_slots_and_wanted_rows():
    rng = np.random.default_rng(1)
    r = fake_runner()
    t0, t1 = table(rng, 4), table(rng, 2)
    entries = [StepEntry(1, 30, [7, 8, 9, 10], [t0], [0, 3]), StepEntry(6, 0, [5], [t1], [0])]
    updates = r._table_updates(entries)
    lay = MetaLayout(5, 2, 3, 4, 1, 0)
    host, facts = r._fill(lay, entries, updates)
    o = lay.offsets
    assert host[o["token_ids"][0]:o["token_ids"][1]].tolist() == [7, 8, 9, 10, 5]
    assert host[o["positions"][0]:o["positions"][1]].tolist() == [30, 31, 32, 33, 0]
    assert host[o["q_start"][0]:o["q_start"][1]].tolist() == [0, 4] and host[o["ctx_len"][0]:o["ctx_len"][1]].tolist() == [34, 1]
    assert host[o["logit_rows"][0]:o["logit_rows"][1]].tolist() == [0, 3, 4]
    want_slots = [t0[1] * 16 + 14, t0[1] * 16 + 15, t0[2] * 16, t0[2] * 16 + 1, t1[0] * 16]
    assert host[o["slot_map0"][0]:o["slot_map0"][1]].tolist() == want_slots
    assert facts["host_q_len"] == [4, 1] and facts["host_slots"] == [1, 6]
    gone = StepEntry(1, 34, [1], [[t0[0], t0[1], -1, t0[3]]], [0])    # its page was given back
    with pytest.raises(ValueError, match="given back"):
        r._fill(MetaLayout(1, 1, 1, 1, 1, 0), [gone], [([], [])])


def test_entries_are_checked_before_anything_runs():
    r = fake_runner()
    ok = StepEntry(0, 0, [1, 2], [[0]], [1])
    r._validate([ok])
    for bad, msg in ((StepEntry(0, 0, [], [[0]], []), "without tokens"), (StepEntry(9, 0, [1], [[0]], [0]), "outside the 8"),
                     (StepEntry(0, 0, [1000], [[0]], [0]), "outside the vocabulary"), (StepEntry(0, 0, [1], [[0]], [1]), "wanted place"),
                     (StepEntry(0, 16 * 64, [1], [[0]], [0]), "beyond the")):
        with pytest.raises(ValueError, match=msg):
            r._validate([bad])
    with pytest.raises(ValueError, match="same request"):
        r._validate([ok, StepEntry(0, 5, [3], [[0]], [0])])
