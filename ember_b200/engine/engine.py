"""The engine: requests in, tokens out.  Scheduler above, step function below.

``Engine.step`` asks the scheduler for the next batch, turns it into one model step (prompt
portions beside single decoded tokens), samples on the device for every run that reached the
end of its known tokens, reads the sampled ids back (the step's only device-to-host read) and
commits them.  ``generate`` runs requests to completion on the calling thread (the
reference's synchronous path: src/engine/engine.cpp:662-677).
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence, Union

import torch

from ..sampling import device as device_sampler
from ..sampling.params import SamplingParams
from .batch import StepEntry
from .runner import ModelRunner
from .scheduler import Request, Scheduler, Sequence_


class Engine:
    def __init__(self, runner: ModelRunner, max_batch_tokens: Optional[int] = None, max_seqs: Optional[int] = None,
                 max_prefill_chunk: int = 512, max_context: Optional[int] = None, sampler=None):
        self.runner = runner
        # sampler(logits, params, counters) -> one token id per row; the device kernel by default
        self.sampler = sampler or (lambda lg, ps, cs: device_sampler.sample(lg, ps, cs).cpu().tolist())
        spec = runner.spec
        self.scheduler = Scheduler(
            runner.cache,
            max_batch_tokens=min(max_batch_tokens or runner.max_batch_tokens, runner.max_batch_tokens),
            max_seqs=min(max_seqs or runner.max_requests, runner.max_requests),
            max_prefill_chunk=max_prefill_chunk,
            max_context=min(max_context or spec.max_positions, spec.max_positions),
            eos_ids=spec.eos_ids,
            on_admit=lambda rid: runner.storage.reset_slot(runner.cache.get(rid).slot) if runner.storage else None)
        self._seed_counter = 0x5EED

    # ------------------------------------------------------------------ intake
    def submit(self, request: Request) -> Sequence_:
        if request.sampling.seed == 0 and not request.sampling.greedy:
            self._seed_counter += 1
            seed = ((time.time_ns() * 0x9E3779B97F4A7C15) ^ self._seed_counter) & ((1 << 64) - 1)
            request.sampling = SamplingParams(request.sampling.temperature, request.sampling.top_p,
                                              request.sampling.top_k, request.sampling.min_p, seed or 1)
        return self.scheduler.submit(request, vocab_size=self.runner.spec.vocab_size)

    # -------------------------------------------------------------------- step
    def step(self) -> bool:
        """One scheduling step; False if there was nothing to do."""
        sched = self.scheduler
        batch = sched.schedule()
        if not batch:
            return False
        entries, params, counters = [], [], []
        for seq, n in batch:
            want = ()
            if sched.wants_logits(seq, n):
                want = (n - 1,)
                params.append(seq.request.sampling)
                counters.append(len(seq.tokens))        # position of the token being drawn
            entries.append(StepEntry(seq.id, seq.tokens[seq.computed:seq.computed + n], want))
        try:
            logits = self.runner.step(entries)
            sampled: List[int] = []
            if logits is not None:
                sampled = self.sampler(logits, params, counters)
        except Exception:
            sched.fail_running()
            raise
        sched.commit(batch, sampled)
        return True

    # ---------------------------------------------------------------- generate
    def generate(self, prompts: Union[Sequence[int], Sequence[Sequence[int]]],
                 sampling: Optional[SamplingParams] = None, max_tokens: int = 256, ignore_eos: bool = False,
                 stop_tokens: Sequence[int] = ()) -> Union[List[int], List[List[int]]]:
        """Generated token ids for one prompt (a list of ids) or several (a list of lists); host
        tokens in, host tokens out.  A stop token is not part of the result."""
        single = len(prompts) > 0 and not isinstance(prompts[0], (list, tuple))
        plist = [prompts] if single else list(prompts)
        sampling = sampling or SamplingParams(temperature=0.0)
        seqs = [self.submit(Request(prompt=list(p), sampling=sampling, max_tokens=max_tokens,
                                    ignore_eos=ignore_eos, stop_tokens=tuple(stop_tokens))) for p in plist]
        while any(s.finished is None for s in seqs):
            if not self.step():
                break
        outs = [list(s.output) for s in seqs]
        return outs[0] if single else outs

    @property
    def stats(self):
        return self.scheduler.stats
