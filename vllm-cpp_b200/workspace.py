"""Scratch memory of a step: where the parts' activation buffers come from.

The reference sizes its scratch buffers once, in the engine's constructor
(src/paged_engine.cpp:201-211), and a step allocates nothing.  Here a step that
runs kernel by kernel takes every buffer from a :class:`Workspace` owned by the
model runner, so that no step asks the device allocator for anything once the
workspace has its size.  Parts call :func:`empty` for their outputs; outside a
step that has a workspace (while a CUDA graph is captured, in a kernel test)
this is ``torch.empty``.

A workspace has three regions, each handed out front to back:

* ``step``   -- buffers that live for the whole step (the step's integers, the
  residual stream, the logits); reset when the next step begins, so **what a
  step returns is valid until the next step of the same runner starts**;
* two ``layer`` regions used in turn by the runs of the execution order: run
  ``i`` takes from region ``i % 2``, which is reset when run ``i`` begins.  What
  a run hands to the next one (its pending delta) therefore outlives the run
  that made it by exactly one run, which is as long as it is read.  **Whatever
  several runs share** (the work items an attention part lays out once per step)
  must come from the ``step`` region: make it through ``ctx.plan`` or
  ``ctx.upload``, or inside ``with workspace.whole_step():``.

All work of a step is queued on one stream, so a region may be handed out again
as soon as the host has moved on: the kernels that read the old contents are
ahead in the queue of those that write the new.  A request that does not fit is
served by ``torch.empty`` and remembered; the region is enlarged before the next
step, so sizes settle after the first step of the largest shape (the runner
makes such a step when it is built, if it is told the step token budget).
"""
from __future__ import annotations

import math

import torch

ALIGN = 256
_ELEM = {torch.float32: 4, torch.bfloat16: 2, torch.int32: 4, torch.float16: 2, torch.int64: 8, torch.uint8: 1}

_active: "Workspace | None" = None


class _Region:
    def __init__(self, device):
        self.device = device
        self.buffer = torch.empty(0, dtype=torch.uint8, device=device)
        self.used = 0        # bytes handed out since the last reset
        self.wanted = 0      # bytes asked for since the last reset, served or not
        self.peak = 0        # the most ever asked for between two resets

    def reset(self) -> None:
        self.peak = max(self.peak, self.wanted)
        self.used = self.wanted = 0

    def fit(self) -> bool:
        """Enlarges the buffer to the peak demand; True if it had to."""
        self.peak = max(self.peak, self.wanted)
        if self.peak <= self.buffer.numel():
            return False
        size = (-(-int(self.peak * 1.125) // (1 << 20)) + 4) * (1 << 20)     # an eighth and 4 MB to spare
        self.buffer = torch.empty(size, dtype=torch.uint8, device=self.device)
        return True

    def take(self, shape, dtype):
        n = math.prod(shape) * _ELEM[dtype]
        padded = -(-n // ALIGN) * ALIGN
        at = self.wanted
        self.wanted += padded
        if at != self.used or at + padded > self.buffer.numel():
            return None      # once one request has overflowed, later ones of this round do too (their offsets moved)
        self.used += padded
        return self.buffer[at:at + n].view(dtype).view(shape)


class Workspace:
    def __init__(self, device):
        self.device = torch.device(device)
        self.step_region = _Region(self.device)
        self.layer_regions = (_Region(self.device), _Region(self.device))
        self._current = self.step_region
        self.overflows = 0     # requests that torch.empty had to serve
        self.resizes = 0

    # ---- a step ----
    def __enter__(self):
        global _active
        self._outer = _active
        _active = self
        self.step_region.reset()
        for r in self.layer_regions:
            r.reset()
        for r in (self.step_region,) + self.layer_regions:
            if r.fit():
                self.resizes += 1
        self._current = self.step_region
        return self

    def __exit__(self, *exc):
        global _active
        _active = self._outer
        self._current = self.step_region
        return False

    def begin_run(self, index: int) -> None:
        r = self.layer_regions[index % 2]
        r.reset()
        self._current = r

    def end_runs(self) -> None:
        self._current = self.step_region

    def take(self, shape, dtype) -> torch.Tensor:
        t = self._current.take(tuple(shape), dtype)
        if t is None:
            self.overflows += 1
            t = torch.empty(tuple(shape), dtype=dtype, device=self.device)
        return t

    def bytes(self) -> int:
        return self.step_region.buffer.numel() + sum(r.buffer.numel() for r in self.layer_regions)


def empty(shape, dtype, device) -> torch.Tensor:
    """An uninitialised buffer for an activation: from the running step's workspace, else from torch."""
    if _active is not None and torch.device(device).type == "cuda":
        return _active.take(shape, dtype)
    return torch.empty(tuple(shape), dtype=dtype, device=device)


def zeros(shape, dtype, device) -> torch.Tensor:
    return empty(shape, dtype, device).zero_()


class whole_step:
    """Within this context buffers come from the region that lives for the whole step, whichever run is on."""

    def __enter__(self):
        self._ws = _active
        if self._ws is not None:
            self._saved = self._ws._current
            self._ws._current = self._ws.step_region
        return self

    def __exit__(self, *exc):
        if self._ws is not None:
            self._ws._current = self._saved
        return False


def begin_run(index: int) -> None:
    """Called by the model before run ``index`` of its execution order."""
    if _active is not None:
        _active.begin_run(index)


def end_runs() -> None:
    if _active is not None:
        _active.end_runs()
