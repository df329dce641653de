"""The engine: requests in, tokens out.  Scheduler above, step function below.

``Engine.step`` asks the scheduler for the next batch, turns it into one model step (prompt
portions beside single decoded tokens), samples on the device for every run that reached the
end of its known tokens, reads the sampled ids back (the step's only device-to-host read) and
commits them.  ``generate`` runs requests to completion on the calling thread (the
reference's synchronous path: src/engine/engine.cpp:662-677).

With the device sampler the engine is pipelined by one step: a launched step stays *in flight*
until the next call.  When every running request is decoding, the next step is launched before
the ids of the one in flight have been read: its tokens are references to the sampler's output
buffer on the device (``ModelRunner.sampled_ids``), so the GPU never waits for the host's
scheduling, packing and committing.  What the host could not know at that point is whether a
request stopped on the token in flight; such a request's share of the speculated step is
dropped when that step is committed (its pages were already given back, and whatever the step
still writes into them precedes, in stream order, any later owner's writes).  Everything the
host can foresee (the token limit, the context limit, pages running out, waiting requests,
cancellations) makes the engine commit first and schedule in the ordinary way.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence, Union

import torch

from .. import transfers
from ..sampling import device as device_sampler
from ..sampling.params import SamplingParams
from .batch import StepEntry
from .runner import DeviceError, ModelRunner
from .scheduler import Request, Scheduler, Sequence_


class _InFlight:
    """A launched step whose sampled ids have not been read yet."""

    __slots__ = ("batch", "rows", "host", "event", "err")

    def __init__(self, batch, rows, host, event, err=0):
        self.batch, self.rows, self.host, self.event, self.err = batch, rows, host, event, err


class Engine:
    def __init__(self, runner: ModelRunner, max_batch_tokens: Optional[int] = None, max_seqs: Optional[int] = None,
                 max_prefill_chunk: int = 512, max_context: Optional[int] = None, sampler=None,
                 pipeline: bool = True):
        self.runner = runner
        # sampler(logits, params, counters) -> one token id per row on the host.  A caller's own sampler
        # makes every step synchronous; the device kernel (the default) allows the one-step pipeline.
        self.sampler = sampler
        # (a runner with ``set_sampled_ids`` can be told the ids of a host sampler: the tests' fake model)
        self.pipeline = bool(pipeline) and (sampler is None or hasattr(runner, "set_sampled_ids"))
        self._inflight: Optional[_InFlight] = None
        self._staging: List = []          # pinned buffers for the sampled ids, with their events
        self._staging_at = 0
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
        """One scheduling step; False if there was nothing to do.  In pipelined mode the step launched
        here is committed by the next call (or by ``drain``)."""
        sched = self.scheduler
        did = False
        if self._inflight is not None:
            ahead = self._speculate(self._inflight)     # launched before the ids in flight are read
            self._commit(self._inflight)
            self._inflight = ahead
            if ahead is not None:
                return True
            did = True
        batch = sched.schedule()
        if not batch:
            return did
        entries, params, counters = [], [], []
        for seq, n in batch:
            want = ()
            if sched.wants_logits(seq, n):
                want = (n - 1,)
                params.append(seq.request.sampling)
                counters.append(len(seq.tokens))        # position of the token being drawn
            entries.append(StepEntry(seq.id, seq.tokens[seq.computed:seq.computed + n], want))
        launched = self._launch(batch, entries, params, counters, 0)
        if self.pipeline:
            self._inflight = launched
        else:
            self._commit(launched)
        return True

    def drain(self) -> None:
        """Commits the step in flight, if any."""
        if self._inflight is not None:
            rec, self._inflight = self._inflight, None
            self._commit(rec)

    def _ids_staging(self, rows: int):
        if len(self._staging) < 4:
            # the sampled ids and, in the last place, the kernels' error word (``ModelRunner.ids_and_err``)
            self._staging.append((torch.empty(max(self.runner.max_requests, 1) + 1, dtype=torch.int32, pin_memory=True),
                                  torch.cuda.Event()))
        self._staging_at = (self._staging_at + 1) % len(self._staging)
        return self._staging[self._staging_at]

    def _launch(self, batch, entries, params, counters, n_prev: int) -> _InFlight:
        """Runs the step and the sampler; with the device sampler nothing is read back here."""
        try:
            logits = self.runner.step(entries, n_prev=n_prev) if n_prev else self.runner.step(entries)
            if logits is None:
                return _InFlight(batch, 0, None, None)
            rows = logits.shape[0]
            if self.sampler is not None:
                ids = [int(t) for t in self.sampler(logits, params, counters)]
                if self.pipeline:
                    self.runner.set_sampled_ids(ids)
                # the host sampler has read the logits, so the step is complete: its error word can be read
                read_error = getattr(self.runner, "read_error", None)
                return _InFlight(batch, rows, ids, None, read_error() if read_error else 0)
            device_sampler.sample(logits, params, counters, out=self.runner.sampled_ids[:rows])
            host, event = self._ids_staging(rows)
            host.copy_(self.runner.ids_and_err, non_blocking=True)      # ids and the error word: one small copy
            event.record()
            transfers.add_d2h(4 * host.numel())
            return _InFlight(batch, rows, host, event)
        except Exception:
            self._inflight = None
            self.scheduler.fail_running()
            raise

    def _commit(self, rec: _InFlight) -> None:
        sched = self.scheduler
        sampled: List[int] = []
        code = rec.err
        if rec.rows:
            if rec.event is not None:
                rec.event.synchronize()
                sampled = rec.host[:rec.rows].tolist()
                code = int(rec.host[-1])
            else:
                sampled = rec.host
        if code:
            self._device_failed(code)
        if any(seq.finished is not None for seq, _ in rec.batch):
            # a speculated step holds requests that stopped on the token before it: their share is dropped
            batch, kept, it = [], [], iter(sampled)
            for seq, n in rec.batch:
                tok = next(it) if sched.wants_logits(seq, n) or seq.finished is not None else None
                if seq.finished is None:
                    batch.append((seq, n))
                    if tok is not None:
                        kept.append(tok)
            sched.commit(batch, kept)
            return
        sched.commit(rec.batch, sampled)

    def _device_failed(self, code: int) -> None:
        """A kernel of a committed step set the error word (a token or page id out of range, a bounded wait that
        ran out): the step's tokens cannot be trusted.  Every running request ends with an error, a speculated
        step in flight is dropped, the runner clears the word and the scratch the aborted kernels may have left
        dirty, and the caller gets a ``DeviceError``."""
        self._inflight = None
        self.scheduler.fail_running()
        reset = getattr(self.runner, "reset_after_error", None)
        if reset:
            reset()
        raise DeviceError(ModelRunner.describe_error(code))

    def _speculate(self, rec: _InFlight) -> Optional[_InFlight]:
        """The step after the one in flight, if the host can lay it out without that step's ids: every
        running request is in the step in flight with one token, none of them ends by a limit the host can
        foresee, nobody waits or is cancelled, and each gets its page.  Returns None otherwise."""
        if not self.pipeline or rec.rows == 0:
            return None
        sched = self.scheduler
        batch = rec.batch
        if sched.waiting or len(batch) != len(sched.running) or rec.rows != len(batch):
            return None
        for seq, n in batch:
            if (n != 1 or seq.finished is not None or seq.cancelled or seq.computed + 1 != len(seq.tokens)
                    or seq.generated + 2 > seq.request.max_tokens or len(seq.tokens) + 2 > sched.max_context):
                return None
        cache = self.runner.cache
        for seq, _ in batch:
            if not cache.ensure(seq.id, seq.computed + 2):
                return None          # pages are short: commit first, then the scheduler may preempt
        entries, params, counters = [], [], []
        for row, (seq, _) in enumerate(batch):
            entries.append(StepEntry(seq.id, (-(row + 1),), (0,)))
            params.append(seq.request.sampling)
            counters.append(len(seq.tokens) + 1)        # the token in flight takes position len(tokens)
        return self._launch(list(batch), entries, params, counters, rec.rows)

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
        self.drain()
        outs = [list(s.output) for s in seqs]
        return outs[0] if single else outs

    @property
    def stats(self):
        return self.scheduler.stats
