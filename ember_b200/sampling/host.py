"""Host statement of the sampler: the semantics the device kernel must agree with.

From src/backend/sampling_host.cpp:20-85 and src/backend/sampling_rng.hpp:21-33: temperature,
then top-k (value descending, index ascending), softmax over the kept set in double, top-p
prefix, min-p floor, and a Gumbel-max draw whose noise is a pure function of
(seed, counter, token id) — ``counter`` is the position of the token being drawn, so a request
draws the same tokens whatever shares its batch.
"""
from __future__ import annotations

from typing import List, Tuple

import numpy as np

from .params import GREEDY_THRESHOLD, SamplingParams

_M64 = (1 << 64) - 1


def rng_mix(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def gumbel_noise(seed: int, counter: int, token: int) -> np.float32:
    h = rng_mix((seed & _M64) ^ rng_mix((counter * 0x632BE59BD9B4E019 + token) & _M64))
    u = (np.float32(h >> 40) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)
    return np.float32(-np.log(-np.log(u, dtype=np.float32), dtype=np.float32))


def sampling_distribution(logits: np.ndarray, p: SamplingParams) -> List[Tuple[int, float]]:
    """The kept tokens with their renormalised probabilities, best first."""
    logits = np.asarray(logits, dtype=np.float32)
    if p.temperature <= GREEDY_THRESHOLD:
        return [(int(np.argmax(logits)), 1.0)]
    x = logits / np.float32(p.temperature)
    order = np.lexsort((np.arange(x.size), -x.astype(np.float64)))     # value descending, index ascending
    if 0 < p.top_k < x.size:
        order = order[:p.top_k]
    xs = x[order].astype(np.float64)
    probs = np.exp(xs - xs[0])
    probs /= probs.sum()
    n = len(order)
    if p.top_p < 1.0:
        cum = np.cumsum(probs)
        hit = np.nonzero(cum >= np.float64(np.float32(p.top_p)))[0]
        if hit.size:
            n = int(hit[0]) + 1
    if p.min_p > 0.0:
        floor = np.float64(np.float32(p.min_p)) * probs[0]
        m = 1
        while m < n and probs[m] >= floor:
            m += 1
        n = m
    kept = probs[:n].sum()
    return [(int(order[i]), float(probs[i] / kept)) for i in range(n)]


def sample_host(logits: np.ndarray, p: SamplingParams, counter: int) -> int:
    dist = sampling_distribution(logits, p)
    if len(dist) == 1:
        return dist[0][0]
    logits = np.asarray(logits, dtype=np.float32)
    best, best_score = dist[0][0], -np.inf
    for tok, _ in dist:
        score = np.float32(logits[tok] / np.float32(p.temperature)) + gumbel_noise(p.seed, counter, tok)
        if score > best_score:
            best, best_score = tok, score
    return best
