"""Helpers of the GPU tests: traces for the four ways of cutting the work, and comparison of
replayed logits with the plain implementation."""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import numpy as np


def rel_err(a, b) -> float:
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def trace_whole(requests: Dict[str, List[int]]) -> List[dict]:
    """Each request alone and whole, every position wanted."""
    steps = []
    for i, (rid, toks) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]})
    return steps


def trace_tail_decode(requests: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps, n = [], 0
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        n += 1
        for t in range(head, len(toks)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [toks[t]], "want": [0]}],
                          "end": [rid] if t == len(toks) - 1 else []})
            n += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(requests: Dict[str, List[int]], sizes: Sequence[int] = (7, 2, 19, 3, 33, 2, 16, 5, 64)) -> List[dict]:
    """Portions of changing size, down to two tokens, crossing page edges."""
    steps, n = [], 0
    for rid, toks in requests.items():
        at, k = 0, 0
        while at < len(toks):
            m = min(sizes[k % len(sizes)], len(toks) - at)
            steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[at:at + m], "want": list(range(m))}],
                          "end": [rid] if at + m == len(toks) else []})
            at += m
            k += 1
            n += 1
    return steps


def trace_mixed(requests: Dict[str, List[int]], live: int = 4, seed: int = 0, decode_tail: int = 12,
                max_portion: int = 24) -> List[dict]:
    """Up to ``live`` requests at a time: portions of some beside single tokens of others; a
    request that ends makes room (and pages) for the next."""
    rng = np.random.default_rng(seed)
    waiting = list(requests.items())
    running: List[Tuple[str, List[int], int]] = []
    steps, n = [], 0
    while waiting or running:
        while waiting and len(running) < live:
            rid, toks = waiting.pop(0)
            running.append((rid, toks, 0))
        entries, ended, nxt = [], [], []
        for rid, toks, at in running:
            if rng.random() < 0.15 and len(running) > 1:
                nxt.append((rid, toks, at))          # left out of this step, goes on later
                continue
            left = len(toks) - at
            if left <= decode_tail:
                m = 1
            else:
                m = int(min(left - decode_tail, rng.integers(2, max_portion + 1)))
            entries.append({"id": rid, "tokens": toks[at:at + m], "want": list(range(m))})
            if at + m == len(toks):
                ended.append(rid)
            else:
                nxt.append((rid, toks, at + m))
        running = nxt
        if entries:
            steps.append({"step": n, "entries": entries, "end": ended})
            n += 1
    return steps


def max_live_tokens(steps: List[dict], round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held: Dict[str, int] = {}
    worst = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum((v + round_to - 1) // round_to * round_to for v in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return worst


def collect(steps: List[dict], outputs: Dict[int, np.ndarray]) -> Dict[str, Dict[int, np.ndarray]]:
    """Per request: position -> logits row, from the per-step outputs."""
    at: Dict[str, int] = {}
    got: Dict[str, Dict[int, np.ndarray]] = {}
    for s in steps:
        row = 0
        for e in s["entries"]:
            base = at.get(e["id"], 0)
            for w in e["want"]:
                got.setdefault(e["id"], {})[base + w] = outputs[s["step"]][row]
                row += 1
            at[e["id"]] = base + len(e["tokens"])
        for rid in s["end"]:
            at.pop(rid, None)
    return got


def first_mismatch(got: Dict[str, Dict[int, np.ndarray]], want: Dict[str, np.ndarray], tol: float):
    """(request, position, error) of the first position whose relative error exceeds ``tol``, and the worst error."""
    worst, first = 0.0, None
    for rid, rows in got.items():
        for pos in sorted(rows):
            e = rel_err(rows[pos], want[rid][pos])
            if not np.isfinite(e):
                e = float("inf")
            worst = max(worst, e)
            if e > tol and first is None:
                first = (rid, pos, e)
    return first, worst
