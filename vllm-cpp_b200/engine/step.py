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
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from .. import ops
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
    block_table: torch.Tensor         # int32 [E, max_blocks]
    slot_map: torch.Tensor            # int32 [T]: page * page_size + offset of each token's cache entry


class StepContext:
    """Tensors and counts of one step, shared by all parts."""

    def __init__(self, entries: list[StepEntry], layout: CacheLayout, page_size: int, device, status: torch.Tensor):
        self.device = device
        self.status = status
        self.entries = entries
        E = self.E = len(entries)
        lens = [len(e.tokens) for e in entries]
        T = self.T = int(sum(lens))
        self.host_q_len = lens
        self.host_q_start = [0] * E
        self.host_ctx_len = [e.start_pos + n for e, n in zip(entries, lens)]
        self.host_slots = [e.slot for e in entries]
        token_ids = np.empty(T, dtype=np.int32)
        positions = np.empty(T, dtype=np.int32)
        entry_of = np.empty(T, dtype=np.int32)
        rows = []
        t = 0
        for i, e in enumerate(entries):
            n = lens[i]
            self.host_q_start[i] = t
            token_ids[t:t + n] = e.tokens
            positions[t:t + n] = np.arange(e.start_pos, e.start_pos + n, dtype=np.int32)
            entry_of[t:t + n] = i
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"wanted place {w} is outside the entry's {n} tokens")
                rows.append(t + w)
            t += n
        self.n_rows = len(rows)
        self.host_positions = positions

        n_paged = len(layout.paged)
        max_blocks = [1] * n_paged
        for g in range(n_paged):
            max_blocks[g] = max([1] + [len(e.tables[g]) for e in entries])
        # one packed int32 buffer, one copy to the device
        sizes = [T, T, T, E, E, E, E, max(self.n_rows, 1)]
        for g in range(n_paged):
            sizes += [E * max_blocks[g], T]
        offs = np.concatenate([[0], np.cumsum(sizes)])
        packed = np.zeros(int(offs[-1]), dtype=np.int32)
        packed[offs[0]:offs[1]] = token_ids
        packed[offs[1]:offs[2]] = positions
        packed[offs[2]:offs[3]] = entry_of
        packed[offs[3]:offs[4]] = self.host_q_start
        packed[offs[4]:offs[5]] = lens
        packed[offs[5]:offs[6]] = self.host_ctx_len
        packed[offs[6]:offs[7]] = self.host_slots
        packed[offs[7]:offs[7] + self.n_rows] = rows
        for g in range(n_paged):
            mb = max_blocks[g]
            bt = np.full((E, mb), -1, dtype=np.int32)
            sm = np.empty(T, dtype=np.int32)
            for i, e in enumerate(entries):
                tab = np.asarray(e.tables[g], dtype=np.int32)
                bt[i, :len(tab)] = tab
                pos = positions[self.host_q_start[i]:self.host_q_start[i] + lens[i]]
                blk = pos // page_size
                if len(tab) == 0 or blk.max(initial=0) >= len(tab):
                    raise ValueError(f"entry {i}: the block table of group {g} does not reach position {int(pos.max())}")
                pages = tab[blk]
                if (pages < 0).any():
                    raise ValueError(f"entry {i}: a token would be stored in a page that was given back")
                sm[self.host_q_start[i]:self.host_q_start[i] + lens[i]] = pages * page_size + pos % page_size
            packed[offs[8 + 2 * g]:offs[9 + 2 * g]] = bt.ravel()
            packed[offs[9 + 2 * g]:offs[10 + 2 * g]] = sm
        dev = torch.from_numpy(packed).pin_memory().to(device, non_blocking=True) if device.type == "cuda" \
            else torch.from_numpy(packed)
        self.h2d_bytes = packed.nbytes

        def view(k):
            return dev[int(offs[k]):int(offs[k + 1])]

        self.token_ids, self.positions, self.entry_of_token = view(0), view(1), view(2)
        self.q_start, self.q_len, self.ctx_len, self.slots = view(3), view(4), view(5), view(6)
        self.logit_rows = view(7)[:self.n_rows]
        self.groups: list[GroupContext] = []
        for gi, g in enumerate(layout.groups):
            if g.paged:
                k = g.runtime_index
                self.groups.append(GroupContext(page_size, g.spec.window,
                                                view(8 + 2 * k).view(E, max_blocks[k]), view(9 + 2 * k)))
            else:
                self.groups.append(None)
        self._plans: dict = {}

    def plan(self, key, make):
        """Per-step data that several layers share (built by the first one that asks)."""
        if key not in self._plans:
            self._plans[key] = make()
        return self._plans[key]


class ModelRunner:
    """Owns the model, its device cache and the status word; runs steps."""

    def __init__(self, model, page_size: int, num_pages: int, num_slots: int, dtype: torch.dtype, device):
        self.model = model
        self.device = torch.device(device)
        self.dtype = dtype
        self.page_size = page_size
        self.layout = CacheLayout(model.cache_specs())
        self.cache = DeviceCache(self.layout, page_size, num_pages, num_slots, dtype, self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.vocab_size = model.spec.vocab_size
        self.launches = 0

    def step(self, entries: list[StepEntry], check: bool = True) -> torch.Tensor | None:
        """Runs the entries' tokens as one batch.  Returns logits [wanted rows, vocab] (32-bit, on the
        device) in the order of the entries and of their ``want`` lists, or None if nothing was wanted."""
        if not entries:
            return None
        slots = [e.slot for e in entries]
        if len(set(slots)) != len(slots):
            raise ValueError("two entries of one step belong to the same request")
        for e in entries:
            if not e.tokens:
                raise ValueError("an entry without tokens")
            bad = [t for t in e.tokens if not 0 <= t < self.vocab_size]
            if bad:
                raise ValueError(f"token id {bad[0]} is outside the vocabulary of {self.vocab_size}")
            if e.start_pos + len(e.tokens) > self.model.spec.max_positions:
                raise ValueError(f"position {e.start_pos + len(e.tokens) - 1} is beyond the model's "
                                 f"{self.model.spec.max_positions} positions")
        self.cache.reset_state([e.slot for e in entries if e.start_pos == 0])
        ctx = StepContext(entries, self.layout, self.page_size, self.device, self.status)
        self.last_ctx, self.last_h2d_bytes = ctx, ctx.h2d_bytes
        logits = self.model.forward(ctx, self.cache.views)
        if check:
            ops.check_status(self.status)
        return logits
