"""Which steps replay a captured graph, and padded to what: the runner's decisions, which need no GPU."""
import types

from vllm_cpp_b200.engine.step import ModelRunner, StepEntry


def fake_runner(graphs=True, page_size=16):
    r = types.SimpleNamespace(cuda_graphs=graphs, page_size=page_size, page_sizes=[page_size])
    for name in ("GRAPH_BUCKETS", "PORTION_BUCKETS", "MIXED_SINGLES", "MIXED_PORTIONS", "MIXED_TOKENS"):
        setattr(r, name, getattr(ModelRunner, name))
    for name in ("capture_size", "portion_size", "mixed_size", "rows_capacity", "_mixed_updates", "_portion_updates"):
        setattr(r, name, types.MethodType(getattr(ModelRunner, name), r))
    return r


def entry(n, want="last", slot=0, start=0):
    return StepEntry(slot, start, list(range(n)), [[0] * 64], {"last": [n - 1], "none": [], "all": list(range(n))}[want])


def test_single_tokens_round_up_to_a_power_of_two():
    r = fake_runner()
    assert r.capture_size([entry(1, slot=i) for i in range(5)]) == 8
    assert r.capture_size([entry(1)]) == 1
    assert r.capture_size([entry(1, slot=i) for i in range(257)]) is None
    assert r.capture_size([entry(1), entry(2, slot=1)]) is None
    assert r.capture_size([entry(1, want="none")]) is None            # no logits wanted: not a decoding step
    assert fake_runner(graphs=False).capture_size([entry(1)]) is None


def test_a_lone_portion_rounds_up_to_its_bucket():
    r = fake_runner()
    assert r.portion_size([entry(2)]) == 16
    assert r.portion_size([entry(16, want="none")]) == 16
    assert r.portion_size([entry(17)]) == 32
    assert r.portion_size([entry(512)]) == 512
    assert r.portion_size([entry(513)]) is None
    assert r.portion_size([entry(40, want="all")]) is None            # logits wanted at other places than the last
    assert r.portion_size([entry(40), entry(1, slot=1)]) is None
    assert r.portion_size([entry(1)]) is None
    assert r._portion_updates(64) == 64 // 16 + 2


def test_single_tokens_beside_portions():
    r = fake_runner()
    singles = [entry(1, slot=i) for i in range(5)]
    assert r.mixed_size(singles + [entry(60, slot=9)]) == (8, 96)
    assert r.mixed_size(singles + [entry(56, slot=9)]) == (8, 64)      # 8 slots + 56 tokens fill 64 rows exactly
    assert r.mixed_size([entry(30, slot=1), entry(20, slot=2)]) == (0, 64)     # portions only
    assert r.mixed_size([entry(1, slot=i) for i in range(40)] + [entry(100, slot=50)]) == (64, 192)
    assert r.mixed_size(singles + [entry(300, slot=9)]) is None        # more than 256 rows: kernel by kernel
    assert r.mixed_size([entry(1, slot=i) for i in range(65)] + [entry(10, slot=70)]) is None
    assert r.mixed_size(singles + [entry(10, slot=10 + i) for i in range(5)]) is None   # five portions
    assert r.mixed_size([entry(60, slot=9)] + singles) is None         # single tokens must come first
    assert r.mixed_size(singles + [entry(60, slot=9, want="all")]) is None
    assert r.mixed_size(singles) is None                               # that is a decoding step
    assert r.mixed_size([entry(60)]) is None                           # and that a lone portion
    # a one-token entry without logits (the last token of a portion cut by the budget) takes a single-token slot
    assert r.mixed_size([entry(1, want="none")] + [entry(30, slot=3)]) == (8, 64)


def test_rows_of_logits_a_step_computes():
    r = fake_runner()
    singles = [entry(1, slot=i) for i in range(5)]
    assert r.rows_capacity(singles) == 8
    assert r.rows_capacity(singles + [entry(60, slot=9)]) == 8 + ModelRunner.MIXED_PORTIONS
    assert r.rows_capacity([entry(60)]) == 1
    assert r.rows_capacity([entry(600), entry(700, slot=1, want="none")]) == 1
    assert fake_runner(graphs=False).rows_capacity(singles) == 5
