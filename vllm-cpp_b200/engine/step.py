"""The step function: one batch of (request, its next tokens) through the model.

A step takes entries, each a run of consecutive tokens of one request starting at
the number of tokens that request already has in the cache -- a portion of a
prompt cut anywhere, or one decoded token -- lays all of them on one token axis,
runs every layer once over that axis from the cache, and returns 32-bit logits at
the places asked for.  It schedules nothing and samples nothing.

The reference's PagedEngine::step (src/paged_engine.cpp:245-300) schedules, runs
each request on its own (whole prompt in run_prefill :318, one token in
run_decode :451), samples and detokenises in one call; here those are separate
layers and the batch is processed as one.

What reaches the device each step is one packed int32 buffer (token ids,
positions, per-entry starts and lengths, slots, wanted rows, each group's cache
slot of every token, and the block-table entries that are new since the last
step).  The block tables themselves stay on the device, one row per request slot,
and only grow by those new entries.  A step made of single tokens only (decoding)
has a fixed shape once its entry count is rounded up, so it is captured once per
rounded count as a CUDA graph and replayed afterwards; the launch cost of a few
hundred small kernels would otherwise exceed the time the GPU needs for them.
"""
from __future__ import annotations

import collections
import gc

from dataclasses import dataclass, field

import numpy as np
import torch

from .. import ops, workspace
from ..cache.device_cache import CacheLayout, DeviceCache


@dataclass
class StepEntry:
    """tokens [start_pos, start_pos + len(tokens)) of one request."""
    slot: int
    start_pos: int
    tokens: list
    tables: list                      # per paged group: logical block -> page id (-1: given back)
    want: list = field(default_factory=list)   # places among ``tokens`` whose logits are returned


@dataclass
class GroupContext:
    page_size: int
    window: int
    block_table: torch.Tensor         # int32 [num_slots, max_blocks], device resident, row = request slot
    slot_map: torch.Tensor            # int32 [T]: page * page_size + offset of each token's cache entry, -1: none
    upd_count: torch.Tensor           # int32 [1]
    upd_idx: torch.Tensor             # int32 [U]  flat indices into block_table
    upd_val: torch.Tensor             # int32 [U]
    upd_capacity: int


class StagingRing:
    """Pinned host buffers for the packed integers of a step, used in turn.

    The copy of a pinned buffer to the device is asynchronous: the host may be several steps ahead of the GPU
    (a prompt cut into portions samples nothing, so nothing makes the host wait), and a buffer written again
    before its last copy has run would hand that earlier step the later step's tokens, positions and cache
    slots.  Each buffer therefore carries an event recorded after its copy, and is written only once that
    event has passed; with ``DEPTH`` buffers the host waits only when it is that many steps ahead."""

    def __init__(self, size: int, depth: int = 4):
        self.DEPTH = depth
        self.size = 0
        self._buffers: list[torch.Tensor] = []
        self._events: list = []
        self._next = 0
        self.waits = 0          # times the host had to wait for an earlier copy (a measure of how far it runs ahead)
        self._grow(size)

    def _grow(self, size: int) -> None:
        for ev in self._events:
            if ev is not None:
                ev.synchronize()
        self.size = size
        self._buffers = [torch.empty(size, dtype=torch.int32).pin_memory() for _ in range(self.DEPTH)]
        self._events = [None] * self.DEPTH
        self._next = 0

    def send(self, host: np.ndarray, dev: torch.Tensor) -> None:
        """Queues the copy of ``host`` (int32) into the first ``len(host)`` integers of ``dev`` on the current stream."""
        n = host.shape[0]
        if n > self.size:
            self._grow(max(n, 2 * self.size))
        i = self._next
        self._next = (i + 1) % self.DEPTH
        ev = self._events[i]
        if ev is None:
            ev = self._events[i] = torch.cuda.Event()
        elif not ev.query():
            self.waits += 1
            ev.synchronize()
        buf = self._buffers[i][:n]
        buf.numpy()[:] = host
        dev[:n].copy_(buf, non_blocking=True)
        ev.record()


class MetaLayout:
    """Where each array sits in the packed int32 buffer of a step with T tokens, E entries, R wanted rows,
    U block-table updates per group and G paged groups."""

    def __init__(self, T, E, R, U, G, X=0):
        self.T, self.E, self.R, self.U, self.G, self.X = T, E, R, U, G, X
        names = [("token_ids", T), ("positions", T), ("q_start", E), ("q_len", E), ("ctx_len", E), ("slots", E),
                 ("logit_rows", max(R, 1)), ("user", max(X, 1))]
        for g in range(G):
            names += [(f"slot_map{g}", T), (f"upd_count{g}", 1), (f"upd_idx{g}", max(U, 1)), (f"upd_val{g}", max(U, 1))]
        self.offsets = {}
        off = 0
        for n, size in names:
            self.offsets[n] = (off, off + size)
            off += size
        self.size = off


class StepContext:
    """Tensors and counts of one step, shared by all parts.  ``T`` and ``E`` are the launch sizes (the real
    counts, or the rounded-up counts of a captured step whose extra entries are empty)."""

    def __init__(self, runner, layout: MetaLayout, dev_buffer: torch.Tensor, static: bool):
        self.device = runner.device
        self.status = runner.status
        self._runner = runner
        self.static = static
        self.meta_layout = layout
        self.T, self.E, self.n_rows = layout.T, layout.E, layout.R
        self.buffer = dev_buffer
        v = lambda n: dev_buffer[layout.offsets[n][0]:layout.offsets[n][1]]
        self.token_ids, self.positions = v("token_ids"), v("positions")
        self.q_start, self.q_len, self.ctx_len, self.slots = v("q_start"), v("q_len"), v("ctx_len"), v("slots")
        self.logit_rows = v("logit_rows")[:layout.R]
        self.user = v("user")[:layout.X]      # integers of the caller's own (the sampler's per-row records)
        self.groups = []
        for g in runner.layout.groups:
            if g.paged:
                k = g.runtime_index
                self.groups.append(GroupContext(runner.page_sizes[k], g.spec.window, runner.tables[k], v(f"slot_map{k}"),
                                                v(f"upd_count{k}"), v(f"upd_idx{k}"), v(f"upd_val{k}"), layout.U))
            else:
                self.groups.append(None)
        self._plans: dict = {}
        self._marks: list = []
        # host-side facts of the current step (refreshed by fill)
        self.entries: list[StepEntry] = []
        self.host_q_len, self.host_q_start, self.host_ctx_len, self.host_slots = [], [], [], []

    def upload(self, host: np.ndarray) -> torch.Tensor:
        """An int32 array of the host on the device, for this step.  A captured step does this once, at capture;
        a step that runs kernel by kernel takes the room from the step's workspace and a pinned staging buffer."""
        host = np.ascontiguousarray(host, dtype=np.int32)
        if self.static or self._runner is None:
            return torch.from_numpy(host).to(self.device)
        with workspace.whole_step():
            dev = workspace.empty(host.shape, torch.int32, self.device)
        self._runner.staging.send(host.reshape(-1), dev.view(-1))
        return dev

    def mark(self, label: str) -> None:
        """With profiling on: the kernels launched since the last mark belong to the group ``label`` (an event is
        recorded here; the runner adds up the times between events after the step).  Otherwise nothing."""
        if self._runner is not None and self._runner.profile is not None and not self.static:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._marks.append((label, ev))

    def plan(self, key, make):
        """Per-step data that several layers share (built by the first one that asks; its buffers live as long as
        the step, not only as long as the layer that happened to build it)."""
        if key not in self._plans:
            with workspace.whole_step():
                self._plans[key] = make()
        return self._plans[key]


class ModelRunner:
    """Owns the model, its device cache, the device-resident block tables and the status word; runs steps."""

    GRAPH_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)
    GRAPH_CONTEXT_BOUNDS = (8192,)      # captured steps are kept per context class: up to 8192 tokens, and beyond
    MAX_GRAPHS = 48                     # captured steps kept; the least recently used one goes when another is captured
    PORTION_BUCKETS = (16, 32, 64, 128, 256, 512)   # token counts of captured steps that run one prompt portion
    # captured steps of single tokens beside prompt portions: slots for single-token entries, which come first, then
    # MIXED_PORTIONS slots for portions; MIXED_TOKENS are the token rows of the whole step (the products work in
    # token tiles of up to 256: a step padded to 264 rows would cost two tiles)
    MIXED_SINGLES = (0, 8, 32, 64)
    MIXED_PORTIONS = 4
    MIXED_TOKENS = (32, 64, 96, 128, 192, 256)

    def __init__(self, model, page_size: int, num_pages: int, num_slots: int, dtype: torch.dtype, device,
                 cuda_graphs: bool = True, max_model_len: int | None = None, max_step_tokens: int | None = None,
                 profile: bool = False):
        """``max_step_tokens``: the most tokens a step will bring; given, the scratch memory of steps that run
        kernel by kernel is sized now (by running the model over that many padding rows), so that no later step
        allocates.  Without it the scratch grows to what the steps need as they come."""
        self.model = model
        self.device = torch.device(device)
        self.dtype = dtype
        self.page_size = page_size
        self.num_slots = num_slots
        self.layout = CacheLayout(model.cache_specs())
        self.cache = DeviceCache(self.layout, page_size, num_pages, num_slots, dtype, self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.vocab_size = model.spec.vocab_size
        self.max_positions = min(max_model_len or model.spec.max_positions, model.spec.max_positions)
        n_paged = len(self.layout.paged)
        # each paged group has pages of its own size (the engine's unless its caches asked for another)
        self.page_sizes = [self.layout.page_size_of(g, page_size) for g in self.layout.paged]
        self.max_blocks = [-(-self.max_positions // ps) for ps in self.page_sizes]
        self.tables = [torch.full((num_slots, mb), -1, dtype=torch.int32, device=self.device) for mb in self.max_blocks]
        self._uploaded = [[0] * num_slots for _ in range(n_paged)]   # table entries of each slot already on the device
        # profiling: milliseconds per group of kernels, summed over the steps so far (None: off); a profiled runner
        # runs every step kernel by kernel, since the events sit between the kernels
        self.profile: dict | None = {} if profile else None
        self.profile_steps = 0
        self.cuda_graphs = (cuda_graphs and not profile and self.device.type == "cuda" and getattr(model, "capturable", True))
        self._graphs: collections.OrderedDict[tuple, tuple] = collections.OrderedDict()   # least recently used first
        self.last_ctx = None
        self.last_h2d_bytes = 0
        self.workspace = workspace.Workspace(self.device)
        self.staging = StagingRing(4096, depth=16)     # for steps that run kernel by kernel (a captured step has its own)
        # (a model with a part that reads host-side facts of a step cannot run over padding: its scratch grows on demand)
        if max_step_tokens and self.device.type == "cuda" and getattr(model, "capturable", True):
            self.size_workspace(max_step_tokens)
        self.graph_replays = 0
        self.launches_per_graph: dict[tuple, int] = {}

    # ------------------------------------------------------------------ host side of a step
    def _validate(self, entries):
        slots = [e.slot for e in entries]
        if len(set(slots)) != len(slots):
            raise ValueError("two entries of one step belong to the same request")
        for e in entries:
            if not e.tokens:
                raise ValueError("an entry without tokens")
            if not 0 <= e.slot < self.num_slots:
                raise ValueError(f"slot {e.slot} is outside the {self.num_slots} request slots")
            if min(e.tokens) < 0 or max(e.tokens) >= self.vocab_size:
                bad = [t for t in e.tokens if not 0 <= t < self.vocab_size][0]
                raise ValueError(f"token id {bad} is outside the vocabulary of {self.vocab_size}")
            if e.start_pos + len(e.tokens) > self.max_positions:
                raise ValueError(f"position {e.start_pos + len(e.tokens) - 1} is beyond the {self.max_positions} "
                                 f"positions this engine was set up for")
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise ValueError(f"wanted place {w} is outside the entry's {len(e.tokens)} tokens")

    def _table_updates(self, entries):
        """Per paged group: (flat indices, values) of block-table entries the device does not have yet."""
        ups = []
        for g in range(len(self.tables)):
            idx, val = [], []
            for e in entries:
                if e.start_pos == 0:
                    self._uploaded[g][e.slot] = 0     # a request that starts (again) from nothing
                tab = e.tables[g]
                have = self._uploaded[g][e.slot]
                need = -(-(e.start_pos + len(e.tokens)) // self.page_sizes[g])
                if need > len(tab):
                    raise ValueError(f"the block table of group {g} does not reach position "
                                     f"{e.start_pos + len(e.tokens) - 1}")
                for b in range(have, need):
                    idx.append(e.slot * self.max_blocks[g] + b)
                    val.append(tab[b])
                self._uploaded[g][e.slot] = max(have, need)
            ups.append((idx, val))
        return ups

    def _fill(self, lay: MetaLayout, entries, updates):
        """Packs the step into one host int32 array following the layout; also returns the host-side facts."""
        packed = np.zeros(lay.size, dtype=np.int32)
        o = lay.offsets
        E = len(entries)
        lens = [len(e.tokens) for e in entries]
        starts = np.concatenate([[0], np.cumsum(lens)])[:-1].astype(np.int32) if E else np.zeros(0, np.int32)
        T = int(sum(lens))
        tok = packed[o["token_ids"][0]:o["token_ids"][1]]
        pos = packed[o["positions"][0]:o["positions"][1]]
        rows = []
        for i, e in enumerate(entries):
            s, n = int(starts[i]), lens[i]
            tok[s:s + n] = e.tokens
            pos[s:s + n] = np.arange(e.start_pos, e.start_pos + n, dtype=np.int32)
            rows += [s + w for w in e.want]
        packed[o["q_start"][0]:o["q_start"][0] + E] = starts
        packed[o["q_start"][0] + E:o["q_start"][1]] = T          # empty padding entries start at the end
        packed[o["q_len"][0]:o["q_len"][0] + E] = lens
        packed[o["ctx_len"][0]:o["ctx_len"][0] + E] = [e.start_pos + n for e, n in zip(entries, lens)]
        packed[o["slots"][0]:o["slots"][0] + E] = [e.slot for e in entries]
        packed[o["logit_rows"][0]:o["logit_rows"][0] + len(rows)] = rows
        for g in range(len(self.tables)):
            ps = self.page_sizes[g]
            sm = packed[o[f"slot_map{g}"][0]:o[f"slot_map{g}"][1]]
            sm[:] = -1
            for i, e in enumerate(entries):
                s, n = int(starts[i]), lens[i]
                tab = np.asarray(e.tables[g], dtype=np.int64)
                p = np.arange(e.start_pos, e.start_pos + n)
                pages = tab[p // ps]
                if (pages < 0).any():
                    raise ValueError("a token would be stored in a page that was given back")
                sm[s:s + n] = pages * ps + p % ps
            idx, val = updates[g]
            if len(idx) > lay.U:
                raise RuntimeError("internal: more block-table updates than the step's buffer holds")
            packed[o[f"upd_count{g}"][0]] = len(idx)
            packed[o[f"upd_idx{g}"][0]:o[f"upd_idx{g}"][0] + len(idx)] = idx
            packed[o[f"upd_val{g}"][0]:o[f"upd_val{g}"][0] + len(idx)] = val
        facts = dict(entries=entries, host_q_len=lens, host_q_start=[int(s) for s in starts],
                     host_ctx_len=[e.start_pos + n for e, n in zip(entries, lens)],
                     host_slots=[e.slot for e in entries])
        return packed, facts

    def _apply_table_updates(self, ctx: StepContext):
        """What a step does on the device before the model runs: new block-table entries, and the initial state of
        requests that start in this step."""
        self.cache.reset_state(ctx)
        for k, table in enumerate(self.tables):
            g = next(gc for gc, grp in zip(ctx.groups, self.layout.groups) if grp.paged and grp.runtime_index == k)
            if g.upd_capacity:
                ops.scatter_i32(table, g.upd_idx, g.upd_val, g.upd_count, g.upd_capacity)

    def reset_tables(self) -> None:
        """Forgets which block-table entries the device holds.  A request normally (re)starts at position 0,
        which does this for its slot; call this when slots are handed to requests that start further on."""
        self._uploaded = [[0] * self.num_slots for _ in self.tables]

    def capture_size(self, entries) -> int | None:
        """The padded entry count of the captured step that would run these entries, or None if they run
        kernel by kernel (prompt portions, rows wanted other than one per entry, graphs switched off)."""
        if not self.cuda_graphs or not entries:
            return None
        if not all(len(e.tokens) == 1 and len(e.want) == 1 for e in entries):
            return None
        return next((b for b in self.GRAPH_BUCKETS if b >= len(entries)), None)

    def portion_size(self, entries) -> int | None:
        """The padded token count of the captured step that would run these entries: one entry, a prompt portion of
        up to 512 tokens, logits wanted at most at its last token.  Kernel by kernel the host needs some twenty
        microseconds a launch, which for a short portion is twice the time the GPU needs."""
        if not self.cuda_graphs or len(entries) != 1:
            return None
        e = entries[0]
        n = len(e.tokens)
        if n < 2 or n > self.PORTION_BUCKETS[-1] or e.want not in ([], [n - 1]):
            return None
        return next(b for b in self.PORTION_BUCKETS if b >= n)

    def mixed_size(self, entries) -> tuple[int, int] | None:
        """(single-token slots, token rows) of the captured step that would run these entries: single-token
        entries first, then one to four prompt portions of two tokens or more with logits wanted at their last
        token or nowhere, up to 64 single tokens and 256 tokens in all (beyond that the GPU needs longer for a step
        than the host needs to launch it kernel by kernel).  None: they run kernel by kernel."""
        if not self.cuda_graphs or len(entries) < 2:
            return None
        n_single = 0
        while n_single < len(entries) and len(entries[n_single].tokens) == 1:
            n_single += 1
        portions = entries[n_single:]
        if not portions or len(portions) > self.MIXED_PORTIONS or n_single > self.MIXED_SINGLES[-1]:
            return None
        tokens = 0
        for e in portions:
            n = len(e.tokens)
            if n < 2 or e.want not in ([], [n - 1]):
                return None
            tokens += n
        singles = next(b for b in self.MIXED_SINGLES if b >= n_single)
        rows = next((b for b in self.MIXED_TOKENS if b >= singles + tokens), None)
        return None if rows is None else (singles, rows)

    def _mixed_updates(self, singles: int, rows: int) -> int:
        """Block-table entries that a captured mixed step's buffer has room for."""
        return singles + (rows - singles) // min(self.page_sizes + [self.page_size]) + 2 * self.MIXED_PORTIONS

    def rows_capacity(self, entries) -> int:
        """Rows of logits that the step running these entries computes: the wanted ones, or more where a captured
        step rounds up (the caller sizes what it sends along per row by this)."""
        n_rows = sum(len(e.want) for e in entries)
        bucket = self.capture_size(entries)
        if bucket:
            return bucket
        mixed = self.mixed_size(entries)
        if mixed:
            return mixed[0] + self.MIXED_PORTIONS
        return n_rows

    def _portion_updates(self, portion: int) -> int:
        """Block-table entries that a captured portion's buffer has room for: the pages its tokens can touch."""
        return portion // min(self.page_sizes + [self.page_size]) + 2

    # ------------------------------------------------------------------ running
    def step(self, entries: list[StepEntry], check: bool = True, user=None, post=None, post_key=None):
        """Runs the entries' tokens as one batch.  Returns logits [wanted rows, vocab] (32-bit, on the
        device) in the order of the entries and of their ``want`` lists, or None if nothing was wanted.
        The returned tensor of a decoding step is reused by the next such step: copy what must outlive it.

        ``user``: int32 numbers of the caller's own, carried to the device with the step's buffer (``ctx.user``).
        ``post(ctx, logits)``: work to run right after the model on the same stream (sampling); its result is
        returned instead of the logits.  A captured step includes it, so ``post_key`` must name everything about
        it that changes which kernels it launches."""
        if not entries:
            return None
        self._validate(entries)
        updates = self._table_updates(entries)
        n_rows = sum(len(e.want) for e in entries)
        bucket = self.capture_size(entries)
        portion = None if bucket else self.portion_size(entries)
        if bucket and all(len(u[0]) <= bucket for u in updates) and (post is None or post_key is not None):
            logits = self._step_graph(entries, updates, bucket, user, post, post_key)
        elif (portion and all(len(u[0]) <= self._portion_updates(portion) for u in updates)
              and (post is None or post_key is not None)):
            logits = self._step_portion_graph(entries, updates, portion, n_rows, user, post, post_key)
        elif (not bucket and (mixed := self.mixed_size(entries)) and (post is None or post_key is not None)
              and all(len(u[0]) <= self._mixed_updates(*mixed) for u in updates)):
            logits = self._step_mixed_graph(entries, updates, mixed, n_rows, user, post, post_key)
        else:
            logits = self._step_eager(entries, updates, n_rows, user, post)
        if check:
            ops.check_status(self.status)
        return logits

    def _step_eager(self, entries, updates, n_rows, user=None, post=None):
        T = sum(len(e.tokens) for e in entries)
        U = max([len(u[0]) for u in updates] + [0])
        lay = MetaLayout(T, len(entries), n_rows, U, len(self.tables), 0 if user is None else len(user))
        host, facts = self._fill(lay, entries, updates)
        if user is not None:
            host[lay.offsets["user"][0]:lay.offsets["user"][0] + len(user)] = user
        with self.workspace, ops.hold_stream():   # kernel by kernel, the host's time per launch is what a short portion waits for
            dev = workspace.empty((lay.size,), torch.int32, self.device)
            self.staging.send(host, dev)
            ctx = StepContext(self, lay, dev, static=False)
            ctx.__dict__.update(facts)
            self.last_ctx, self.last_h2d_bytes = ctx, host.nbytes
            ctx.mark("start")
            self._apply_table_updates(ctx)
            ctx.mark("tables")
            logits = self.model.forward(ctx, self.cache.views)
            result = post(ctx, logits) if post is not None else logits
            if post is not None:
                ctx.mark("sampling")
            if self.profile is not None:
                self._add_up(ctx)
            return result

    def _add_up(self, ctx) -> None:
        """Adds the times between the step's marks to the totals of their groups (waits for the step to end)."""
        torch.cuda.current_stream().synchronize()
        for (_, a), (label, b) in zip(ctx._marks, ctx._marks[1:]):
            self.profile[label] = self.profile.get(label, 0.0) + a.elapsed_time(b)
        self.profile_steps += 1

    def size_workspace(self, max_step_tokens: int) -> None:
        """Sizes the scratch memory for steps of up to ``max_step_tokens`` tokens: the model runs over padding rows
        (token 0, stored nowhere, entries of length 0: nothing is read or written in the cache), once per token
        count at which the parts' buffers are largest -- the budget itself, and the largest counts whose products
        still write partial sums per k-slice."""
        sizes = sorted({max_step_tokens, min(max_step_tokens, 1024), min(max_step_tokens, 128)})
        for T in sizes:
            # as many single-token entries as there are request slots (their contexts taken as the longest there
            # can be, which gives their key ranges the most slices), the rest of the rows one portion; logits
            # wanted of every entry, and room for the integers a sampler sends along
            S = min(self.num_slots, T)
            E = S + (1 if T > S else 0)
            lay = MetaLayout(T, E, E, E + T // min(self.page_sizes + [self.page_size]) + 2, len(self.tables), 8 * E + T)
            host = np.zeros(lay.size, dtype=np.int32)
            for g in range(len(self.tables)):
                host[lay.offsets[f"slot_map{g}"][0]:lay.offsets[f"slot_map{g}"][1]] = -1
            q_len = [1] * S + ([T - S] if T > S else [])
            q_start = list(range(S)) + ([S] if T > S else [])
            ctx_len = [self.max_positions] * S + ([T - S] if T > S else [])
            for _ in range(2):     # the first pass finds the sizes, the second must fit
                with self.workspace, ops.hold_stream():
                    dev = workspace.empty((lay.size,), torch.int32, self.device)
                    self.staging.send(host, dev)
                    ctx = StepContext(self, lay, dev, static=False)
                    ctx.entries, ctx.host_q_len, ctx.host_q_start, ctx.host_ctx_len, ctx.host_slots = [], q_len, q_start, ctx_len, [0] * E
                    self.model.forward(ctx, self.cache.views)
        torch.cuda.current_stream().synchronize()
        ops.check_status(self.status)

    USER_INTS_PER_ENTRY = 12  # room in a captured step's buffer for the caller's numbers

    def _fill_decode(self, lay: MetaLayout, entries, updates, user):
        """_fill for single-token entries, without per-entry array work."""
        E, B = len(entries), lay.E
        pad = B - E
        toks = [e.tokens[0] for e in entries]
        pos = [e.start_pos for e in entries]
        parts = [toks, [0] * pad, pos, [0] * pad, list(range(E)), [E] * pad, [1] * E, [0] * pad,
                 [p + 1 for p in pos], [0] * pad, [e.slot for e in entries], [0] * pad,
                 list(range(E)), [0] * pad]
        ux = [0] * max(lay.X, 1)
        if user is not None:
            ux[:len(user)] = [int(v) for v in user]
        parts.append(ux)
        for g in range(len(self.tables)):
            sm, ps = [], self.page_sizes[g]
            for e, p in zip(entries, pos):
                page = e.tables[g][p // ps]
                if page < 0:
                    raise ValueError("a token would be stored in a page that was given back")
                sm.append(page * ps + p % ps)
            idx, val = updates[g]
            n = len(idx)
            parts += [sm, [-1] * pad, [n], idx, [0] * (lay.U - n), val, [0] * (lay.U - n)]
        flat = [x for part in parts for x in part]
        assert len(flat) == lay.size, (len(flat), lay.size)
        facts = dict(entries=entries, host_q_len=[1] * E, host_q_start=list(range(E)),
                     host_ctx_len=[p + 1 for p in pos], host_slots=[e.slot for e in entries])
        return np.asarray(flat, dtype=np.int32), facts

    def _graph(self, key):
        self._graphs.move_to_end(key)
        return self._graphs[key]

    def _keep_graph(self, key, captured) -> None:
        self._graphs[key] = captured
        while len(self._graphs) > self.MAX_GRAPHS:
            old, _ = self._graphs.popitem(last=False)   # its buffers go back to the allocator with the graph
            self.launches_per_graph.pop(old, None)

    def _replay(self, key, host, facts, nbytes):
        """Copies a filled step buffer to the device and replays the captured step of ``key``; returns its result."""
        graph, ctx, result, staging = self._graph(key)
        ctx.__dict__.update(facts)
        staging.send(host, ctx.buffer)
        self.last_ctx, self.last_h2d_bytes = ctx, nbytes
        graph.replay()
        self.graph_replays += 1
        ops.launch_count += self.launches_per_graph[key]
        return result

    def _fill_padded(self, key, entries, updates, user):
        """_fill into the layout of the captured step of ``key``, with the caller's integers."""
        lay = self._graphs[key][1].meta_layout
        if user is not None and len(user) > lay.X:
            raise ValueError(f"a captured step carries at most {lay.X} user integers, {len(user)} given")
        host, facts = self._fill(lay, entries, updates)
        if user is not None:
            host[lay.offsets["user"][0]:lay.offsets["user"][0] + len(user)] = user
        return host, facts

    def _step_graph(self, entries, updates, bucket, user=None, post=None, post_key=None):
        # one captured step per padded batch size and context class: the attention part slices the key ranges of
        # short contexts differently from long ones, and a captured step cannot ask how long they are
        longest = max(e.start_pos for e in entries) + 1
        ctx_bound = next((b for b in self.GRAPH_CONTEXT_BOUNDS if longest <= b), None)
        key = (bucket, post_key if post is not None else None, ctx_bound)
        if key not in self._graphs:
            self._capture(key, post)
        lay = self._graphs[key][1].meta_layout
        if user is not None and len(user) > lay.X:
            raise ValueError(f"a captured step carries at most {lay.X} user integers, {len(user)} given")
        host, facts = self._fill_decode(lay, entries, updates, user)
        return self._replay(key, host, facts, host.nbytes)[:len(entries)]

    def _step_portion_graph(self, entries, updates, portion, n_rows, user=None, post=None, post_key=None):
        """One prompt portion through a captured step of ``portion`` token rows: the tokens beyond the entry's own
        are padding (token 0 at position 0, stored nowhere, attended by nothing, their rows never read)."""
        key = ("portion", portion, n_rows, post_key if post is not None else None)
        if key not in self._graphs:
            self._capture_portion(key, post)
        host, facts = self._fill_padded(key, entries, updates, user)
        return self._replay(key, host, facts, host.nbytes)

    def _step_mixed_graph(self, entries, updates, mixed, n_rows, user=None, post=None, post_key=None):
        """Single tokens beside prompt portions through a captured step: the single-token entries fill the first
        slots (token row = slot, as in a captured decoding step), unused slots stay empty, the portions follow."""
        singles, rows = mixed
        n_single = sum(1 for e in entries if len(e.tokens) == 1)
        longest = max([e.start_pos + 1 for e in entries[:n_single]] + [1])
        ctx_bound = next((b for b in self.GRAPH_CONTEXT_BOUNDS if longest <= b), None)
        key = ("mixed", singles, rows, post_key if post is not None else None, ctx_bound)
        if key not in self._graphs:
            self._capture_mixed(key, post)
        empty = StepEntry(0, 0, [], [[] for _ in self.tables], [])
        slotted = entries[:n_single] + [empty] * (singles - n_single) + entries[n_single:]
        host, facts = self._fill_padded(key, slotted, updates, user)
        result = self._replay(key, host, facts, host.nbytes)
        return None if result is None else result[:n_rows]

    def _capture_graph(self, key, lay, host_facts, post, ctx_bound=None, logit_rows=None):
        """Captures the forward pass (and what ``post`` adds) over a static step buffer of layout ``lay``.  The
        capture itself runs on empty entries (length 0), which store nothing and attend to nothing; ``host_facts``
        are the entry lengths that the attention part lays its work items out for."""
        dev = torch.zeros(lay.size, dtype=torch.int32, device=self.device)
        staging = StagingRing(lay.size)
        ctx = StepContext(self, lay, dev, static=True)
        ctx.static_max_ctx = ctx_bound
        host = np.zeros(lay.size, dtype=np.int32)
        o = lay.offsets
        for g in range(len(self.tables)):
            host[o[f"slot_map{g}"][0]:o[f"slot_map{g}"][1]] = -1
        if logit_rows is not None:
            host[o["logit_rows"][0]:o["logit_rows"][1]] = logit_rows
        dev.copy_(torch.from_numpy(host))
        ctx.host_q_len, ctx.host_q_start, ctx.host_ctx_len, ctx.host_slots = host_facts

        def run():
            self._apply_table_updates(ctx)
            logits = self.model.forward(ctx, self.cache.views)
            return post(ctx, logits) if post is not None else logits

        # warm up on a side stream (library handles, lazy module loads), then capture
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            run()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        before = ops.launch_count
        graph = torch.cuda.CUDAGraph()
        # Nothing may be destroyed on the device while a capture is open: a captured graph of an engine that is no
        # longer referenced, finalised by the collector in the middle of this capture, makes the capture invalid.
        # So the collector rests until the capture is closed; what is garbage goes at its next turn after that.
        # (Collecting here instead costs a tenth of a second and more per capture in a process with a large heap.)
        collecting = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(graph):
                result = run()
        finally:
            if collecting:
                gc.enable()
        self.launches_per_graph[key] = ops.launch_count - before
        self._keep_graph(key, (graph, ctx, result, staging))

    def _capture_mixed(self, key, post=None):
        """``singles`` one-token entries and MIXED_PORTIONS portions in ``rows`` token rows together.  The attention
        part lays out work items for every slot: sliced key ranges for the single tokens, query tiles over all the
        remaining rows for each portion; at replay the kernels leave out empty slots and cut the portions' items
        down to the tokens that are there."""
        _, singles, T, _, ctx_bound = key
        P = self.MIXED_PORTIONS
        E = R = singles + P
        tokens = T - singles
        lay = MetaLayout(T, E, R, self._mixed_updates(singles, T), len(self.tables), 8 * R + T)
        facts = ([1] * singles + [tokens] * P, list(range(singles)) + [singles] * P, [0] * singles + [tokens] * P, [0] * E)
        self._capture_graph(key, lay, facts, post, ctx_bound)

    def _capture_portion(self, key, post=None):
        """One entry of ``portion`` tokens.  The attention part lays its work items out for all ``portion`` tokens;
        at replay the kernels cut them down to the tokens that are there."""
        _, portion, n_rows, _ = key
        lay = MetaLayout(portion, 1, n_rows, self._portion_updates(portion), len(self.tables), 8 * max(n_rows, 1) + portion)
        self._capture_graph(key, lay, ([portion], [0], [portion], [0]), post)

    def _capture(self, key, post=None):
        """``bucket`` single-token entries, each with logits wanted."""
        bucket = key[0]
        lay = MetaLayout(bucket, bucket, bucket, bucket, len(self.tables), bucket * self.USER_INTS_PER_ENTRY)
        facts = ([1] * bucket, list(range(bucket)), [0] * bucket, [0] * bucket)
        self._capture_graph(key, lay, facts, post, key[2], logit_rows=np.arange(bucket))
