"""The scheduler's decisions: admission, portions under a token budget, decoding first, finishing and freeing,
and what happens when pages run out (the youngest running request is preempted and recomputed)."""
import pytest

from vllm_cpp_b200.runtime import runtime


def make(num_pages=16, page=4, seqs=4, budget=8, max_len=64, window=0):
    rt = runtime()
    groups = [rt.GroupSpec(page, num_pages, 0)] + ([rt.GroupSpec(page, num_pages, window)] if window else [])
    return rt, rt.Scheduler(groups, seqs, budget, max_len)


def greedy(rt):
    return rt.SamplingParams(0.0, 1.0, 1.0, 0)


def run(s, token=lambda rid, step: 1000 + step, max_steps=500):
    """Drives the scheduler with made-up tokens; returns the list of steps as [(request, start, n, sample)]."""
    steps = []
    for _ in range(max_steps):
        if not s.has_unfinished():
            break
        out = s.schedule()
        steps.append([(e.request, e.start_pos, len(e.tokens), e.sample) for e in out.entries])
        s.update([token(e.request, e.gen_step) for e in out.entries if e.sample])
        s.cache().check_invariants()
    assert not s.has_unfinished()
    return steps


def test_prompt_is_cut_into_portions_under_the_budget():
    rt, s = make(budget=8)
    a = s.submit(list(range(20)), 3, greedy(rt), [])
    steps = run(s)
    assert steps[:3] == [[(a, 0, 8, False)], [(a, 8, 8, False)], [(a, 16, 4, True)]]      # the last portion samples
    assert steps[3:] == [[(a, 20, 1, True)], [(a, 21, 1, True)]]
    r = s.request(a)
    assert r.generated == [1000, 1001, 1002] and r.finish_reason == "length" and r.state == rt.RequestState.FINISHED
    assert s.cache().free_pages(0) == 16 and s.cache().free_slots() == 4                  # given back at once


def test_decoding_requests_go_first_and_newcomers_fill_the_rest():
    rt, s = make(budget=8, num_pages=32)
    a = s.submit([1, 2, 3], 10, greedy(rt), [])
    s.schedule(); s.update([7])                       # a is decoding now
    b = s.submit(list(range(30)), 2, greedy(rt), [])
    out = s.schedule()
    got = [(e.request, e.start_pos, len(e.tokens), e.sample, e.is_prompt) for e in out.entries]
    assert got == [(a, 3, 1, True, False), (b, 0, 7, False, True)]                      # 1 decoded token + 7 of the budget
    assert out.num_generation_tokens == 1 and out.num_prompt_tokens == 7
    assert list(out.entries[0].tokens) == [7]                                              # the sampled token is fed back
    s.update([8])
    out = s.schedule()
    assert [(e.request, e.start_pos, len(e.tokens)) for e in out.entries] == [(a, 4, 1), (b, 7, 7)]
    s.update([9])


def test_first_come_first_admitted_up_to_the_slot_limit():
    rt, s = make(seqs=2, budget=64, num_pages=64)
    ids = [s.submit([1] * 5, 2, greedy(rt), []) for _ in range(4)]
    out = s.schedule()
    assert [e.request for e in out.entries] == ids[:2] and s.num_waiting() == 2 and s.num_running() == 2
    s.update([5, 5])
    out = s.schedule()
    assert [e.request for e in out.entries] == ids[:2]       # no slot free yet
    s.update([5, 5])                                          # both finish (max_new 2)
    out = s.schedule()
    assert [e.request for e in out.entries] == ids[2:]
    s.update([5, 5])


def test_stop_ids_and_model_length():
    rt, s = make(max_len=12)
    a = s.submit([1, 2, 3], 9, greedy(rt), [42])
    steps = run(s, token=lambda rid, step: 42 if step == 2 else 5)
    assert s.request(a).generated == [5, 5, 42] and s.request(a).finish_reason == "stop"
    b = s.submit([1, 2, 3], 9, greedy(rt), [])
    run(s)
    assert len(s.request(b).generated) == 9 and s.request(b).finish_reason == "length"
    with pytest.raises(ValueError, match="max_model_len"):
        s.submit([1] * 10, 5, greedy(rt), [])
    with pytest.raises(ValueError, match="empty"):
        s.submit([], 5, greedy(rt), [])


def test_a_request_too_large_for_the_empty_pool_is_refused_at_submit():
    rt, s = make(num_pages=4, page=4, max_len=64)
    with pytest.raises(ValueError, match="does not fit"):
        s.submit([1] * 10, 10, greedy(rt), [])
    assert s.submit([1] * 10, 6, greedy(rt), []) == 0


def test_when_pages_run_out_the_youngest_is_preempted_and_recomputed():
    rt, s = make(num_pages=6, page=4, seqs=3, budget=16, max_len=24)
    a = s.submit([1] * 7, 12, greedy(rt), [])           # grows to 19 tokens = 5 pages
    b = s.submit([2] * 7, 12, greedy(rt), [])
    events = []
    tokens = {}
    for _ in range(200):
        if not s.has_unfinished():
            break
        out = s.schedule()
        events.append((list(out.preempted), [(e.request, e.start_pos, len(e.tokens)) for e in out.entries]))
        s.update([100 * (e.request + 1) + e.gen_step for e in out.entries if e.sample])
        s.cache().check_invariants()
    assert not s.has_unfinished()
    preempted = [p for ev in events for p in ev[0]]
    assert preempted and set(preempted) == {b}                       # never the older one
    assert s.request(a).preempt_count == 0 and s.request(b).preempt_count >= 1
    # after a preemption b is fed again from position 0 with prompt + what it had generated
    i = next(k for k, ev in enumerate(events) if ev[0])
    later = [e for ev in events[i + 1:] for e in ev[1] if e[0] == b]
    assert later[0][1] == 0 and later[0][2] > 7
    # no preemption to admit: while a ran alone with b waiting, a was never disturbed
    assert s.request(a).generated == [100 + k for k in range(12)]
    assert s.request(b).generated == [200 + k for k in range(12)]   # the sample index runs on across the recompute
    st = s.stats()
    assert st.preemptions == len(preempted) and st.recomputed_tokens > 0 and st.generated_tokens == 24
    assert s.cache().free_pages(0) == 6


def test_nothing_is_preempted_to_admit_a_newcomer():
    rt, s = make(num_pages=4, page=4, seqs=4, budget=16, max_len=16)
    a = s.submit([1] * 9, 3, greedy(rt), [])            # 3 pages now, 3 at the end
    s.schedule(); s.update([5])
    b = s.submit([2] * 8, 2, greedy(rt), [])            # needs 2 pages now: only 1 is free
    out = s.schedule()
    assert out.preempted == [] and [e.request for e in out.entries] == [a]
    s.update([5])
    out = s.schedule(); s.update([5])                   # a finishes and frees its pages
    out = s.schedule()
    assert [e.request for e in out.entries] == [b] and out.entries[0].sample      # the whole prompt fits the budget
    s.update([5])
    assert s.num_running() == 1


def test_abort_and_protocol_errors():
    rt, s = make()
    a = s.submit([1, 2, 3], 5, greedy(rt), [])
    s.schedule()
    with pytest.raises(Exception, match="before update"):
        s.schedule()
    s.abort(a)                                          # between schedule() and update(): the entry is dropped
    assert s.update([9]) == []
    assert s.request(a).finish_reason == "abort" and s.cache().free_pages(0) == 16
    with pytest.raises(Exception, match="without a scheduled step"):
        s.update([])
    b = s.submit([1, 2, 3], 5, greedy(rt), [])
    s.schedule()
    with pytest.raises(ValueError, match="asked for one"):
        s.update([])
    s.update([1])
    with pytest.raises(Exception, match="unfinished"):
        s.forget(b)
    s.forget(a)
    assert not s.knows(a)


def test_window_group_lets_long_requests_fit_a_small_pool():
    rt, s = make(num_pages=40, page=4, budget=8, max_len=160, window=10)
    a = s.submit([1] * 100, 50, greedy(rt), [])         # 150 tokens: 38 pages in the full group, ~6 in the windowed one
    run(s)
    assert len(s.request(a).generated) == 50
    assert s.cache().free_pages(0) == 40 and s.cache().free_pages(1) == 40


@pytest.mark.parametrize("seed", range(6))
def test_random_workloads_keep_every_promise(seed):
    """Random arrivals, lengths, pools, budgets and windows: every step stays under the token budget and the slot
    limit, a request's tokens arrive in order without gaps, a preempted request starts again from position 0 and is
    fed its prompt and what it had generated, every request ends with exactly the tokens it was promised, and the
    pool is whole again at the end."""
    import random
    rnd = random.Random(seed)
    page = rnd.choice([2, 4, 8])
    window = rnd.choice([0, 0, 6, 16])
    num_pages, seqs, budget = rnd.randint(12, 40), rnd.randint(2, 5), rnd.randint(4, 24)
    max_len = page * num_pages
    rt, s = make(num_pages=num_pages, page=page, seqs=seqs, budget=budget, max_len=max_len, window=window)
    pending = []
    for _ in range(rnd.randint(8, 20)):
        n_prompt = rnd.randint(1, max(1, max_len // 3))
        pending.append((list(rnd.randrange(100) for _ in range(n_prompt)), rnd.randint(1, max(1, max_len // 4))))
    want, fed, next_pos, preemptions = {}, {}, {}, 0
    for step in range(5000):
        if pending and rnd.random() < 0.4:
            prompt, max_new = pending.pop()
            try:
                rid = s.submit(prompt, max_new, greedy(rt), [])
                want[rid] = (prompt, max_new)
                fed[rid], next_pos[rid] = [], 0
            except Exception as e:      # a request that an empty pool could not hold is refused, and says so
                assert "pool" in str(e) or "length" in str(e) or "positions" in str(e), e
        if not s.has_unfinished():
            if not pending:
                break
            continue
        out = s.schedule()
        preemptions += len(out.preempted)
        for rid in out.preempted:
            fed[rid], next_pos[rid] = [], 0                      # recomputed from its first token
        assert sum(len(e.tokens) for e in out.entries) <= budget
        assert len({e.request for e in out.entries}) == len(out.entries) <= seqs
        assert len({e.slot for e in out.entries}) == len(out.entries)
        for e in out.entries:
            assert e.start_pos == next_pos[e.request] and len(e.tokens) >= 1
            fed[e.request] += list(e.tokens)
            next_pos[e.request] += len(e.tokens)
            prompt, _ = want[e.request]
            so_far = prompt + list(s.request(e.request).generated)
            assert fed[e.request] == so_far[:len(fed[e.request])]          # prompt, then what was generated, in order
            assert e.sample == (next_pos[e.request] == len(so_far))         # logits are wanted at the sequence's end only
        s.update([1000 + e.gen_step for e in out.entries if e.sample])
        s.cache().check_invariants()
    assert not s.has_unfinished() and not pending
    for rid, (prompt, max_new) in want.items():
        r = s.request(rid)
        room = max_len - len(prompt)
        assert r.state == rt.RequestState.FINISHED
        assert list(r.generated) == [1000 + i for i in range(min(max_new, room))], (rid, r.finish_reason)
    c = s.cache()
    assert c.free_slots() == seqs and all(c.free_pages(g) == num_pages for g in range(c.num_groups()))
