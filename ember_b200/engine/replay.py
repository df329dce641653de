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
        r = self.runner
        step = record["step"]
        entries = []
        for e in record.get("entries", []):
            rid = e["id"]
            toks = list(e["tokens"])
            if not r.cache.has(rid):
                if not r.admit(rid):
                    raise ReplayError(f"step {step}: no free request slot for {rid!r} "
                                      f"({len(r.cache.live_requests())} requests are live)")
            if not r.reserve(rid, len(toks)):
                raise ReplayError(
                    f"step {step}: the cache pool ({r.cache.capacity_tokens()} tokens) has no pages for "
                    f"{len(toks)} more tokens of {rid!r}; live requests hold {r.cache.used_pages()} pages")
            entries.append(StepEntry(rid, toks, list(e.get("want", []))))
        out = None
        if entries:
            logits = r.step(entries)
            if logits is not None:
                out = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                out.tofile(os.path.join(self.out_dir, f"{step}.f32"))
            r.check_device()
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
