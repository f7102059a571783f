"""The work items the attention part lays out for a step (host-side decisions; no GPU needed)."""
import types

import torch

from vllm_cpp_b200.parts import attention as A


def ctx(q_lens, ctx_lens, static=False, bound=None):
    c = types.SimpleNamespace(device=torch.device("cpu"), host_q_len=list(q_lens), host_ctx_len=list(ctx_lens), static=static)
    starts, s = [], 0
    for n in q_lens:
        starts.append(s)
        s += n
    c.host_q_start = starts
    if static:
        c.static_max_ctx = bound
    return c


def test_single_tokens_get_key_slices_that_fill_the_sms():
    # one request, 4,096 keys: short contexts are cut into at most SHORT_SLICES slices
    p = A.AttentionPlan(ctx([1], [4096]), 32, 8, A.MMA_DECODE_ROWS, A.MMA_SPAN_ROWS)
    assert p.n_dec == 1 and p.nslices == A.SHORT_SLICES and p.n_span_items == 0
    assert p.dec_items.shape == (p.nslices, 6)
    assert p.dec_items[:, 3].tolist() == list(range(p.nslices)) and set(p.dec_items[:, 4].tolist()) == {p.nslices}
    # a long context: as many slices as keep one wave of blocks resident, 128 keys a slice at least
    p = A.AttentionPlan(ctx([1], [32768]), 32, 8, A.MMA_DECODE_ROWS, A.MMA_SPAN_ROWS)
    assert p.nslices == (A.BLOCKS_PER_SM * 148) // 8
    # sixty-four requests: one block per request and KV head already fills the SMs
    p = A.AttentionPlan(ctx([1] * 64, [4096] * 64), 32, 8, A.MMA_DECODE_ROWS, A.MMA_SPAN_ROWS)
    assert p.nslices == 1 and p.dec_rows.tolist() == list(range(64))
    # very short contexts are not cut below 128 keys a slice
    p = A.AttentionPlan(ctx([1], [200]), 32, 8, A.MMA_DECODE_ROWS, A.MMA_SPAN_ROWS)
    assert p.nslices == 1


def test_a_captured_step_slices_for_its_context_class():
    short = A.AttentionPlan(ctx([1] * 8, [0] * 8, static=True, bound=8192), 32, 8, A.MMA_DECODE_ROWS, A.MMA_SPAN_ROWS)
    long = A.AttentionPlan(ctx([1] * 8, [0] * 8, static=True, bound=None), 32, 8, A.MMA_DECODE_ROWS, A.MMA_SPAN_ROWS)
    assert short.nslices == min(A.SHORT_SLICES, (A.BLOCKS_PER_SM * 148) // 64) and long.nslices == (A.BLOCKS_PER_SM * 148) // 64
    assert short.slice_counters.numel() == 8 * 8 and int(short.slice_counters.abs().sum()) == 0


def test_portions_are_cut_into_query_tiles_longest_first():
    # 4 query heads a KV head: 32 tokens fill the 128 rows of a tile
    p = A.AttentionPlan(ctx([100, 1, 40], [1000, 500, 40]), 32, 8, A.MMA_DECODE_ROWS, A.MMA_SPAN_ROWS)
    assert p.n_dec == 1 and p.dec_rows.tolist() == [100]
    items = p.span_items.tolist()
    assert p.n_span_items == len(items) == 4 + 2
    covered = {0: [], 2: []}
    for e, q0, nq, s, ns, _ in items:
        assert (s, ns) == (0, 1) and nq <= 32
        covered[e] += list(range(q0, q0 + nq))
    assert sorted(covered[0]) == list(range(100)) and sorted(covered[2]) == list(range(40))
    # the item that reads the most keys comes first
    reach = [({0: 1000, 2: 40}[e] - {0: 100, 2: 40}[e]) + q0 + nq for e, q0, nq, *_ in items]
    assert reach == sorted(reach, reverse=True)
    # seven query heads a KV head: 18 tokens a tile (126 rows)
    p = A.AttentionPlan(ctx([40], [40]), 14, 2, A.MMA_DECODE_ROWS, A.MMA_SPAN_ROWS)
    assert sorted(i[2] for i in p.span_items.tolist()) == [4, 18, 18]


def test_key_slices_that_merge_in_clusters_are_chosen_so_that_all_clusters_run_at_once(monkeypatch):
    """Where the decode kernel can merge a token's slices within a cluster of blocks, the number of slices is the
    largest (eight at most; six where two blocks share an SM) of which the device runs as many clusters at once as
    there are (request, KV head) pairs.  The device's answers here are a B200's."""
    alone = {1: 148, 2: 74, 3: 45, 4: 33, 5: 26, 6: 22, 7: 15, 8: 15}        # clusters of blocks with an SM each
    shared = {1: 296, 2: 148, 3: 93, 4: 71, 5: 56, 6: 45, 7: 37, 8: 33}     # two blocks an SM
    asked = []

    def fits(hd, size, deep):
        asked.append((hd, size, deep))
        return (alone if deep else shared)[size]

    monkeypatch.setattr(A.ops, "attn_mma_max_clusters", fits)
    monkeypatch.setattr(A.ops, "num_sms", lambda: 148)

    def plan(batch, context=4096, **kw):
        return A.AttentionPlan(ctx([1] * batch, [context] * batch, **kw), 32, 8, A.MMA_DECODE_ROWS, A.MMA_SPAN_ROWS, 128)

    want = {1: 8,      # 8 pairs: fifteen clusters of eight fit
            2: 6,      # 16 pairs: not fifteen clusters of eight or seven, but twenty-two of six
            3: 5,      # 24 pairs: twenty-six clusters of five
            4: 6,      # 32 pairs, 192 blocks, two to an SM: forty-five clusters of six (eight would start late)
            8: 4,      # 64 pairs: no more than four slices fill the SMs; seventy-one clusters of four fit
            16: 2}
    for batch, slices in want.items():
        p = plan(batch)
        assert (p.nslices, p.cluster) == (slices, slices), (batch, p.nslices, p.cluster)
    assert all(hd == 128 for hd, _, _ in asked)
    # one slice needs no cluster; long contexts keep their many slices and the merge through global memory
    p = plan(64)
    assert (p.nslices, p.cluster) == (1, 0)
    p = plan(1, 32768)
    assert p.nslices == (A.BLOCKS_PER_SM * 148) // 8 and p.cluster == 0
    # a captured step of the short context class chooses the same way; of the long class, no clusters
    assert plan(8, 0, static=True, bound=8192).cluster == 4
    assert plan(8, 0, static=True, bound=None).cluster == 0
    # without a kernel that merges in clusters (no head size given) nothing changes
    p = A.AttentionPlan(ctx([1], [4096]), 32, 8, A.MMA_DECODE_ROWS, A.MMA_SPAN_ROWS)
    assert (p.nslices, p.cluster) == (A.SHORT_SLICES, 0)
    # a device that takes no clusters of any size: the slices stay, merged through global memory
    monkeypatch.setattr(A.ops, "attn_mma_max_clusters", lambda hd, size, deep: -1)
    p = plan(1)
    assert (p.nslices, p.cluster) == (A.SHORT_SLICES, 0)


def test_many_single_tokens_go_to_the_blocks_that_walk_the_pairs(monkeypatch):
    """More (token, KV head) pairs than resident blocks, no key slices, and short contexts: known in a step that runs
    kernel by kernel, implied by the number of pairs in a captured one."""
    monkeypatch.setattr(A.ops, "num_sms", lambda: 148)
    plan = lambda n, c, **kw: A.AttentionPlan(ctx([1] * n, [c] * n, **kw), 32, 8, A.MMA_DECODE_ROWS, A.MMA_SPAN_ROWS)
    assert A.stream_pays(plan(64, 512), 8) and A.stream_pays(plan(256, 128), 8) and A.stream_pays(plan(40, 2048), 8)
    assert not A.stream_pays(plan(64, 4096), 8)          # long contexts: a block a pair is as fast and ends raggedly
    assert not A.stream_pays(plan(32, 512), 8)           # 256 pairs: a block each is resident at once
    assert not A.stream_pays(plan(64, 512), 2)           # 128 pairs
    assert plan(64, 512).longest == 512 and plan(64, 0, static=True, bound=8192).longest is None
    assert A.stream_pays(plan(256, 0, static=True, bound=8192), 8)
    assert not A.stream_pays(plan(64, 0, static=True, bound=8192), 8) and not A.stream_pays(plan(128, 0, static=True, bound=8192), 8)
    monkeypatch.setattr(A, "STREAM_DECODE", 0)
    assert not A.stream_pays(plan(256, 128), 8)
