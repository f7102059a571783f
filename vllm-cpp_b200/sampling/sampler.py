"""Choosing next tokens from logits, on the device.

Options and their defaults are the reference's: temperature 0.7, top-p 0.8 and a
repetition penalty of 1.1 over everything the request has seen so far
(src/config.h:97-99; src/model.cpp:1291-1352; history = prompt + generated in the
engine path, src/paged_engine.cpp:544-549).  temperature <= 0 is greedy
(src/mlx_backend.cpp:516-524).  A request's draw at generated-token index ``step``
depends only on (seed, step) and its logits, so a request that was preempted and
recomputed continues with the same tokens.

The occurrence counts behind the penalty are per-request state of fixed size:
one row of ``[slots, vocab]`` int32 per state slot, cleared when a request's
first tokens arrive, bumped for every token fed to the model.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass

import numpy as np
import torch

from .. import ops, workspace


@dataclass(frozen=True)
class SamplingOptions:
    temperature: float = 0.7
    top_p: float = 0.8
    repeat_penalty: float = 1.1
    seed: int = 0


def _f2i(x: float) -> int:
    return struct.unpack("<i", struct.pack("<f", float(x)))[0]


class Sampler:
    def __init__(self, vocab_size: int, num_slots: int, device):
        self.vocab, self.num_slots, self.device = vocab_size, num_slots, torch.device(device)
        self.counts = None   # allocated when the first request with a penalty shows up

    def _need_counts(self):
        if self.counts is None:
            self.counts = torch.zeros((self.num_slots, self.vocab), dtype=torch.int32, device=self.device)

    def forget(self, slots: list[int]) -> None:
        """Clears the counts of slots whose requests start (again) from their first token."""
        if slots and self.counts is not None:
            for s in slots:     # a fill per row: no index tensor to allocate
                self.counts[s].zero_()

    @staticmethod
    def token_slots(entries, penalised_slots: set) -> list[int]:
        """For every token of the step: its request's slot + 1 if that request has a penalty, else 0."""
        out = []
        for e in entries:
            out += [e.slot + 1 if e.slot in penalised_slots else 0] * len(e.tokens)
        return out

    def observe(self, token_ids: torch.Tensor, token_slots_plus1: torch.Tensor, n: int) -> None:
        """Counts the step's tokens into their requests' rows; everything is on the device, so a captured step
        can include it."""
        self._need_counts()
        ops.count_tokens(token_ids, token_slots_plus1, self.counts, n, slot_bias=1)

    @staticmethod
    def records(options: list[SamplingOptions], steps: list[int], slots: list[int]):
        """Per-row records for the kernel as a flat list of int32 (8 per row), and the two facts that decide which
        kernels run: whether any row has a penalty (needs the count table), whether no row cuts a nucleus."""
        flat, use_counts, no_nucleus = [], False, True
        for o, step, slot in zip(options, steps, slots):
            pen = o.repeat_penalty if o.repeat_penalty and o.repeat_penalty > 0 else 1.0
            use_counts |= pen != 1.0
            no_nucleus &= (not o.temperature > 0) or o.top_p >= 1.0
            seed = int(o.seed) & 0xFFFFFFFFFFFFFFFF
            lo, hi, st = seed & 0xFFFFFFFF, seed >> 32, step & 0xFFFFFFFF
            flat += [_f2i(o.temperature), _f2i(o.top_p), _f2i(pen), slot if pen != 1.0 else -1,
                     lo - (1 << 32) if lo >= (1 << 31) else lo, hi - (1 << 32) if hi >= (1 << 31) else hi,
                     st - (1 << 32) if st >= (1 << 31) else st, 0]
        return flat, use_counts, no_nucleus

    def sample_records(self, logits: torch.Tensor, params: torch.Tensor, use_counts: bool, no_nucleus: bool) -> torch.Tensor:
        """One token per row of ``logits`` from records already on the device (int32 [rows, 8])."""
        if use_counts:
            self._need_counts()
        out = workspace.empty((logits.shape[0],), torch.int32, self.device)
        ops.sample(logits, params, self.counts if use_counts else None, out, no_nucleus)
        return out

    def sample(self, logits: torch.Tensor, options: list[SamplingOptions], steps: list[int], slots: list[int]) -> torch.Tensor:
        """One token per row of ``logits``; returns int32 [rows] on the device."""
        flat, use_counts, no_nucleus = self.records(options, steps, slots)
        params = torch.tensor(flat, dtype=torch.int32).view(-1, 8).to(self.device)
        return self.sample_records(logits, params, use_counts, no_nucleus)
