"""Trace replay: feeds given token ids through the model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives the same
``ModelRunner`` (model, step function, cache manager, kernels) that generation uses.

Input, one JSON object a line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step run as one batch.  For a step in which something is wanted the logits at
the wanted places are written to ``<out>/<step>.f32`` as little-endian float32 [wanted, vocab],
in the order of the entries and of ``want``.  After every step a line ``done <step>`` is
printed and flushed.
"""
from __future__ import annotations

import json
import os
import sys
from typing import IO, Iterable, Optional

import numpy as np

from .batch import StepEntry
from .runner import ModelRunner


class ReplayError(RuntimeError):
    pass


class TraceReplayer:
    def __init__(self, runner: ModelRunner, out_dir: str):
        self.runner = runner
        self.out_dir = out_dir
        os.makedirs(out_dir, exist_ok=True)

    def run_step(self, record: dict) -> Optional[np.ndarray]:
        """Runs one record.  A step with more tokens than the runner takes at once is run as several
        batches, cut at the limit (the logits at a position do not depend on where a step is cut)."""
        r = self.runner
        step = record["step"]
        todo = []                                  # [id, tokens, {offset in tokens: [output rows]}]
        seen = set()
        n_out = 0
        for e in record.get("entries", []):
            rid = e["id"]
            toks = list(e["tokens"])
            if rid in seen:
                raise ReplayError(f"step {step}: request {rid!r} appears twice")
            seen.add(rid)
            want = {}
            for w in e.get("want", []):
                if not (0 <= int(w) < len(toks)):
                    raise ReplayError(f"step {step}: request {rid!r} wants row {w} of {len(toks)} tokens")
                want.setdefault(int(w), []).append(n_out)
                n_out += 1
            if not toks:
                continue
            if not r.cache.has(rid):
                if not r.admit(rid):
                    raise ReplayError(f"step {step}: no free request slot for {rid!r} "
                                      f"({len(r.cache.live_requests())} requests are live)")
            if not r.reserve(rid, len(toks)):
                raise ReplayError(
                    f"step {step}: the cache pool ({r.cache.capacity_tokens()} tokens) has no pages for "
                    f"{len(toks)} more tokens of {rid!r}; live requests hold {r.cache.used_pages()} pages")
            todo.append((rid, toks, want))
        out = None
        limit = r.max_batch_tokens
        at, offset = 0, 0                          # next entry and how much of it has run
        while at < len(todo):
            entries, rows, room = [], [], limit
            while at < len(todo) and room > 0:
                rid, toks, want = todo[at]
                n = min(room, len(toks) - offset)
                here = sorted(w for w in want if offset <= w < offset + n)
                for w in here:
                    rows.append(want[w])
                entries.append(StepEntry(rid, toks[offset:offset + n], [w - offset for w in here]))
                room -= n
                offset += n
                if offset == len(toks):
                    at, offset = at + 1, 0
            logits = r.step(entries)
            if logits is not None:
                got = logits.detach().to("cpu").numpy()
                if out is None:
                    out = np.empty((n_out, got.shape[1]), dtype="<f4")
                for i, dest in enumerate(rows):
                    out[dest] = got[i]             # a place wanted twice is written twice
            r.check_device()
        if out is not None:
            out.tofile(os.path.join(self.out_dir, f"{step}.f32"))
        for rid in record.get("end", []):
            if r.cache.has(rid):
                r.release(rid)
        return out

    def run(self, lines: Iterable[str], log: IO = sys.stdout) -> int:
        n = 0
        for line in lines:
            line = line.strip()
            if not line:
                continue
            record = json.loads(line)
            self.run_step(record)
            print(f"done {record['step']}", file=log, flush=True)
            n += 1
        return n
