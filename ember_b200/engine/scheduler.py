"""Continuous batching: which requests run in the next step, with how many tokens each.

Policy, as the reference's (src/engine/engine.cpp:226-357, 389-436):

1. running requests that are decoding (one token to compute) come first;
2. then running requests still reading their prompt get a portion,
   ``min(need, budget left, max_prefill_chunk)`` tokens;
3. then waiting requests are admitted in arrival order while the token budget, the request
   limit and the pages allow (not in a step that preempted someone).

When pages run out for a running request, the *newest* running request that is not already in
this step's batch is preempted: all its pages go back, its computed count returns to zero, and
it waits at the front of the queue to be recomputed (prompt and generated tokens as one
prompt); if none can be preempted the request itself is.  Sampling is a pure function of
(seed, position), so a recomputed request continues with the same tokens.

The scheduler owns no model: it talks to a ``CacheManager`` and hands out (request, count)
pairs; ``Engine`` turns them into a step.
"""
from __future__ import annotations

import itertools
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence, Tuple

from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams

FINISH_STOP, FINISH_LENGTH, FINISH_CANCELLED, FINISH_ERROR = "stop", "length", "cancelled", "error"


@dataclass
class Request:
    """What a caller submits (src/engine/engine.hpp:35-42)."""

    prompt: Sequence[int]
    sampling: SamplingParams = field(default_factory=SamplingParams)
    max_tokens: int = 256
    ignore_eos: bool = False
    stop_tokens: Sequence[int] = ()
    tag: str = ""


@dataclass
class Sequence_:
    id: int
    request: Request
    tokens: List[int]
    prompt_len: int
    computed: int = 0
    generated: int = 0
    finished: Optional[str] = None
    cancelled: bool = False
    preemptions: int = 0
    output: List[int] = field(default_factory=list)   # delivered tokens (a stop token is not delivered)


@dataclass
class SchedulerStats:
    steps: int = 0
    requests_done: int = 0
    prompt_tokens: int = 0
    generated_tokens: int = 0
    preemptions: int = 0


class Scheduler:
    def __init__(self, cache: CacheManager, max_batch_tokens: int = 2048, max_seqs: int = 64,
                 max_prefill_chunk: int = 512, max_context: int = 4096, eos_ids: Sequence[int] = (),
                 on_admit=None):
        self.cache = cache
        self.max_batch_tokens = max_batch_tokens
        self.max_seqs = min(max_seqs, cache.max_requests)
        self.max_prefill_chunk = max(1, min(max_prefill_chunk, max_batch_tokens))
        self.max_context = min(max_context, cache.capacity_tokens())
        self.eos_ids = tuple(eos_ids)
        self.on_admit = on_admit           # called with the request id when it gets its slot
        self.waiting: Deque[Sequence_] = deque()
        self.running: List[Sequence_] = []
        self.stats = SchedulerStats()
        self._ids = itertools.count(1)

    # ------------------------------------------------------------------ intake
    def submit(self, request: Request, vocab_size: Optional[int] = None) -> Sequence_:
        prompt = [int(t) for t in request.prompt]
        if not prompt:
            raise ValueError("the prompt is empty")
        if len(prompt) >= self.max_context:
            raise ValueError(f"the prompt has {len(prompt)} tokens; the context limit is {self.max_context}")
        if vocab_size is not None:
            for t in prompt:
                if not (0 <= t < vocab_size):
                    raise ValueError(f"token id {t} is out of range")
        request.max_tokens = max(1, int(request.max_tokens))
        seq = Sequence_(id=next(self._ids), request=request, tokens=prompt, prompt_len=len(prompt))
        self.waiting.append(seq)
        return seq

    def idle(self) -> bool:
        return not self.waiting and not self.running

    # --------------------------------------------------------------- scheduling
    def _preempt(self, seq: Sequence_) -> None:
        self.cache.release(seq.id)          # pages and the state slot; it is admitted anew later
        seq.computed = 0
        seq.preemptions += 1
        self.stats.preemptions += 1

    def _finish(self, seq: Sequence_, reason: str) -> None:
        seq.finished = reason
        if self.cache.has(seq.id):
            self.cache.release(seq.id)
        self.stats.requests_done += 1

    def schedule(self) -> List[Tuple[Sequence_, int]]:
        """The next step's (request, token count) pairs; empty if there is nothing to run.
        Pages for the chosen tokens are reserved."""
        batch: List[Tuple[Sequence_, int]] = []
        in_batch = set()
        budget = self.max_batch_tokens

        # cancelled requests first: their pages are needed
        for seq in [s for s in self.running if s.cancelled]:
            self.running.remove(seq)
            self._finish(seq, FINISH_CANCELLED)
        for seq in [s for s in self.waiting if s.cancelled]:
            self.waiting.remove(seq)
            self._finish(seq, FINISH_CANCELLED)

        preempted = False
        for decode_pass in (True, False):
            i = 0
            while i < len(self.running) and budget > 0:
                seq = self.running[i]
                need = len(seq.tokens) - seq.computed
                if need <= 0 or (need == 1) != decode_pass:
                    i += 1
                    continue
                n = min(need, budget, self.max_prefill_chunk)
                ok = self.cache.ensure(seq.id, seq.computed + n)
                while not ok:
                    victim = self.running[-1]
                    if victim is seq or victim.id in in_batch:
                        break
                    self._preempt(victim)
                    self.running.pop()
                    self.waiting.appendleft(victim)
                    preempted = True
                    ok = self.cache.ensure(seq.id, seq.computed + n)
                if not ok:
                    self._preempt(seq)
                    self.running.pop(i)
                    self.waiting.appendleft(seq)
                    preempted = True
                    continue
                batch.append((seq, n))
                in_batch.add(seq.id)
                budget -= n
                i += 1

        while not preempted and self.waiting and budget > 0 and len(self.running) < self.max_seqs:
            seq = self.waiting[0]
            fresh = not self.cache.has(seq.id)
            if fresh:
                if self.cache.admit(seq.id) is None:
                    break
                if self.on_admit:
                    self.on_admit(seq.id)
            need = len(seq.tokens) - seq.computed
            n = min(need, budget, self.max_prefill_chunk)
            if not self.cache.ensure(seq.id, seq.computed + n):
                # not even this portion fits: give back what was taken and wait
                self.cache.release(seq.id)
                if not self.running and not batch:
                    # nothing else holds pages, so waiting cannot help: the pool is too small
                    self.waiting.popleft()
                    self._finish(seq, FINISH_ERROR)
                    continue
                break
            self.waiting.popleft()
            self.running.append(seq)
            batch.append((seq, n))
            in_batch.add(seq.id)
            budget -= n
        return batch

    # ----------------------------------------------------------------- results
    def wants_logits(self, seq: Sequence_, n: int) -> bool:
        """A run's last row is sampled from when it reaches the end of the known tokens."""
        return seq.computed + n == len(seq.tokens)

    def commit(self, batch: List[Tuple[Sequence_, int]], sampled: Sequence[int]) -> List[Sequence_]:
        """Applies a step's outcome: counts advance, sampled tokens are appended, finished requests
        give their pages back.  ``sampled`` holds one token per run that wanted logits, in batch
        order.  Returns the requests that finished."""
        done: List[Sequence_] = []
        it = iter(sampled)
        for seq, n in batch:
            if seq.computed < seq.prompt_len:
                self.stats.prompt_tokens += min(n, seq.prompt_len - seq.computed)
            reached_end = self.wants_logits(seq, n)
            seq.computed += n
            if not reached_end:
                continue
            tok = int(next(it))
            seq.tokens.append(tok)
            seq.generated += 1
            self.stats.generated_tokens += 1
            req = seq.request
            is_stop = tok in self.eos_ids or tok in req.stop_tokens
            reason = None
            if is_stop and not req.ignore_eos:
                reason = FINISH_STOP
            elif seq.generated >= req.max_tokens or len(seq.tokens) >= self.max_context:
                reason = FINISH_LENGTH
            if reason != FINISH_STOP or req.ignore_eos:
                seq.output.append(tok)          # the stop token itself is not delivered
            if reason:
                self.running.remove(seq)
                self._finish(seq, reason)
                done.append(seq)
        self.stats.steps += 1
        return done

    def fail_running(self) -> List[Sequence_]:
        """A step threw: every running request ends with an error and gives its pages back
        (src/engine/engine.cpp:147-163)."""
        failed = list(self.running)
        for seq in failed:
            self._finish(seq, FINISH_ERROR)
        self.running.clear()
        return failed
