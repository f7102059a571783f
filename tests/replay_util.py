"""Builds replay traces (lists of step records for bin/trace_run) and runs them."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent


def round64(n):
    return -(-n // 64) * 64


class Trace:
    def __init__(self):
        self.steps = []          # records for trace_run
        self.wanted = []         # per step: list of (request, position) in output order
        self.live = {}           # request -> tokens held
        self.max_tokens = 64

    def add(self, entries, end=()):
        """entries: list of (request id, tokens, start position, wanted local places)."""
        rec = {"step": len(self.steps), "entries": [], "end": list(end)}
        want = []
        for rid, toks, start, places in entries:
            rec["entries"].append({"id": rid, "tokens": [int(t) for t in toks], "want": [int(p) for p in places]})
            want += [(rid, start + p) for p in places]
            self.live[rid] = start + len(toks)
        self.max_tokens = max(self.max_tokens, sum(round64(n) for n in self.live.values()))
        for rid in end:
            self.live.pop(rid, None)
        self.steps.append(rec)
        self.wanted.append(want)


def whole(requests):
    t = Trace()
    for rid, toks in requests.items():
        t.add([(rid, toks, 0, range(len(toks)))], end=[rid])
    return t


def tail_one_by_one(requests, tail=32):
    t = Trace()
    for rid, toks in requests.items():
        head = max(len(toks) - tail, 1)
        t.add([(rid, toks[:head], 0, range(head))])
        for p in range(head, len(toks)):
            t.add([(rid, toks[p:p + 1], p, [0])], end=[rid] if p == len(toks) - 1 else [])
        if head == len(toks):
            t.add([], end=[rid])
    return t


PORTIONS = [7, 2, 16, 3, 2, 5, 33, 2, 9, 4, 64, 2, 11]


def portions(requests, sizes=PORTIONS, last_only=False):
    """Each request alone, cut into portions of the given sizes in turn; logits wanted everywhere, or
    (last_only) at each portion's last token, which is what a serving step asks for."""
    t = Trace()
    k = 0
    for rid, toks in requests.items():
        p = 0
        while p < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - p)
            k += 1
            t.add([(rid, toks[p:p + n], p, [n - 1] if last_only else range(n))], end=[rid] if p + n == len(toks) else [])
            p += n
    return t


def portions_last(requests):
    return portions(requests, sizes=[7, 2, 16, 3, 40, 5, 33, 2, 100, 17, 64, 130], last_only=True)


def mixed(requests, seed=0, max_live=4, decode_tail=12, last_only=False):
    """Up to max_live requests at a time: the prompt part of each goes in portions of changing size,
    its last tokens one by one, beside the others'; a request sometimes sits a step out; a new
    one starts when one ends, in pages the ended one gave back.  ``last_only``: logits are wanted at each
    entry's last token only and single tokens come first in a step, as a serving step has them."""
    rng = np.random.default_rng(seed)
    t = Trace()
    waiting = list(requests.items())
    live = []   # [rid, toks, pos]
    k = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live.append([rid, toks, 0])
            if rng.random() < 0.5:
                break   # stagger the starts
        entries, ended = [], []
        for item in live:
            rid, toks, pos = item
            if len(live) > 1 and rng.random() < 0.15:
                continue  # left out of this step
            if pos >= len(toks) - decode_tail and pos > 0:
                n = 1
            else:
                n = min(PORTIONS[k % len(PORTIONS)], max(len(toks) - decode_tail - pos, 1))
                k += 1
            n = min(n, len(toks) - pos)
            entries.append((rid, toks[pos:pos + n], pos, [n - 1] if last_only else range(n)))
            item[2] = pos + n
            if item[2] == len(toks):
                ended.append(rid)
        live = [it for it in live if it[0] not in ended]
        if last_only:
            entries.sort(key=lambda en: len(en[1]) != 1)
        t.add(entries, end=ended)
    return t


def mixed_last(requests):
    return mixed(requests, seed=2, last_only=True)


def run_trace(model_dir, dtype, trace, out_dir, page_size, extra_env=None, timeout=900, extra_args=()):
    """Runs bin/trace_run on the trace; returns per-step arrays [wanted, vocab] (None where nothing was wanted)."""
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    text = "".join(json.dumps(s) + "\n" for s in trace.steps)
    env = dict(os.environ)
    env.update(extra_env or {})
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
           "--out", str(out_dir), "--max-tokens", str(trace.max_tokens), "--page-size", str(page_size), *extra_args]
    r = subprocess.run(cmd, input=text, capture_output=True, text=True, env=env, timeout=timeout)
    assert r.returncode == 0, f"trace_run failed ({r.returncode}):\n{r.stdout[-2000:]}\n{r.stderr[-4000:]}"
    done = [l for l in r.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == list(range(len(trace.steps)))
    return out_dir


def read_step(out_dir, step, vocab):
    f = Path(out_dir) / f"{step}.f32"
    if not f.exists():
        return None
    return np.fromfile(f, dtype="<f4").reshape(-1, vocab)
