"""The step function: one model, its cache, and ``step(entries) -> logits``.

``ModelRunner`` is what generation, the benchmark and trace replay all drive.  A step runs
only the tokens it is given, as one batch, against what earlier steps left in the cache, and
returns fp32 logits at the wanted places (the reference's contract:
src/backend/backend.hpp:104-117).  Pages for the new tokens are taken from the cache manager
before the step (``reserve``) and given back by ``release``.
"""
from __future__ import annotations

import os
from typing import Hashable, List, Optional, Sequence

import torch

from .. import ops
from ..cache.manager import CacheManager
from ..cache.storage import CacheStorage, cache_bytes_per_token, state_bytes_per_request
from ..config.registry import load_config
from ..config.spec import ModelSpec
from ..model.causal_lm import CausalLM
from ..parts.base import Runtime
from ..weights.loader import WeightStore
from .batch import BatchError, StepBatch, StepContext, StepEntry, Workspace
from ..runtime import StepPacker

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, got {name}")
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got {name!r}") from None


class DeviceError(RuntimeError):
    pass


class ModelRunner:
    def __init__(self, spec: ModelSpec, store: WeightStore, dtype="bfloat16", device="cuda:0",
                 capacity_tokens: Optional[int] = 4096, max_batch_tokens: int = 2048, max_requests: int = 64,
                 page_tokens: int = 16, cuda_graphs: bool = True, memory_fraction: float = 0.92, cache_bytes: int = 0,
                 max_context: Optional[int] = None):
        """``capacity_tokens``: tokens the cache holds (every paged group gets pages for that many).  None or 0
        sizes it after the weights are on the device: from ``cache_bytes`` if given, else from the device's free
        memory so that ``memory_fraction`` of the whole device is in use (weights, cache and buffers), as the
        reference does (src/backend/cuda/cuda_backend.cu:757-780); never more than ``max_requests`` requests of
        ``max_context`` tokens (default: the model's position limit) could use."""
        if not torch.cuda.is_available():
            raise DeviceError("no CUDA device: this engine runs its model on a B200 only (there is no CPU path)")
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.spec = spec
        self.dtype = parse_dtype(dtype)
        self.rt = Runtime(device=self.device, dtype=self.dtype, page_tokens=page_tokens)
        self.max_batch_tokens = int(max_batch_tokens)
        self.max_requests = int(max_requests)
        self.model = CausalLM(spec).load(store, self.rt)
        if not capacity_tokens or capacity_tokens <= 0:
            capacity_tokens = self._capacity_from_memory(memory_fraction, cache_bytes, page_tokens,
                                                         min(max_context or spec.max_positions, spec.max_positions))
        self.cache = CacheManager(self.model.cache_needs(), page_tokens, int(capacity_tokens), self.max_requests)
        self.storage = CacheStorage(self.cache, self.device, self.dtype)
        self.workspace = Workspace(self.device)
        self._packer = StepPacker()
        # one small buffer holds the sampler's output and, behind it, the kernels' error word, so that the engine
        # reads both back with the step's single device-to-host copy.  ``sampled_ids``: where a sampler may leave
        # a step's ids for the next step to read on the device (a token -(r + 1) of a step names row r); the
        # address is fixed, graphs capture it.  ``err``: bits set by kernels (see ``describe_error``).
        self.ids_and_err = torch.zeros(max(self.max_requests, 1) + 1, dtype=torch.int32, device=self.device)
        self.sampled_ids = self.ids_and_err[:-1]
        self.err = self.ids_and_err[-1:]
        self.steps = 0
        # decode steps (one token per run) are captured into CUDA graphs, one per (runs, wanted rows,
        # context bucket); the reference does the same for its decode steps (src/backend/cuda/cuda_backend.cu:376-454)
        # (only if every part of the model launches nothing but kernels that read their indices on the device:
        # a part that reads a step's host views would have one step's values baked into the graph)
        self.cuda_graphs = bool(cuda_graphs) and self.model.graph_safe
        self.graph_context_bucket = 512
        self.graph_max_runs = 256
        self._graphs = {}
        self._graph_seen = set()
        self.graph_replays = 0
        self._capture_row: Optional[int] = None
        self._captured: Optional[torch.Tensor] = None

    def _capacity_from_memory(self, memory_fraction: float, cache_bytes: int, page_tokens: int, max_context: int) -> int:
        """Tokens of cache that fit: what is free now (the weights are loaded), less the share of the device to
        be left alone, the state slots, and room for the step's buffers (residual, activations, logits)."""
        needs = self.model.cache_needs()
        per_token = cache_bytes_per_token(needs, self.dtype)
        useful = (self.max_requests * max_context + page_tokens - 1) // page_tokens * page_tokens
        if per_token == 0:
            return useful
        if cache_bytes and cache_bytes > 0:
            budget = int(cache_bytes)
        else:
            if not (0.0 < memory_fraction <= 1.0):
                raise ValueError(f"memory_fraction must be in (0, 1], got {memory_fraction}")
            torch.cuda.empty_cache()
            free, total = torch.cuda.mem_get_info(self.device)
            buffers = self.max_batch_tokens * self.spec.hidden_size * 64 + self.max_requests * self.spec.vocab_size * 8 \
                + (512 << 20)
            budget = free - int((1.0 - memory_fraction) * total) - buffers - self.max_requests * state_bytes_per_request(needs)
        tokens = max(0, budget) // per_token // page_tokens * page_tokens
        if tokens < 4 * page_tokens:
            raise DeviceError(f"not enough device memory left for the cache ({max(0, budget) / 2**20:.0f} MiB; a token "
                              f"takes {per_token} bytes)")
        return int(min(tokens, useful))

    # -------------------------------------------------------------- constructors
    @classmethod
    def from_dir(cls, model_dir: str, **kw) -> "ModelRunner":
        """The model class is chosen by config.json's architecture, as everywhere."""
        cfg = load_config(model_dir)
        return cls(cfg.to_model_spec(), WeightStore.from_dir(model_dir), **kw)

    # ------------------------------------------------------------------ requests
    def admit(self, request: Hashable) -> bool:
        rc = self.cache.admit(request)
        if rc is None:
            return False
        self.storage.reset_slot(rc.slot)
        return True

    def reserve(self, request: Hashable, new_tokens: int) -> bool:
        """Pages for ``new_tokens`` more tokens of the request; False if the pool cannot give them."""
        return self.cache.ensure(request, self.cache.get(request).tokens + new_tokens)

    def release(self, request: Hashable) -> None:
        self.cache.release(request)

    def cached_tokens(self, request: Hashable) -> int:
        return self.cache.get(request).tokens

    # ----------------------------------------------------------------- debugging
    def set_capture_hidden(self, on: bool, row: int = -1) -> None:
        """Debugging aid (the reference's Backend::set_capture_hidden, src/backend/backend.hpp:119-122): while on,
        every step records the residual stream of one of its tokens (``row`` among the step's tokens; -1 = the
        last) after the embedding and after every run of the layer schedule, so that a drift against another
        implementation can be traced to the layer where it starts.  Such steps run without CUDA graphs."""
        self._capture_row = int(row) if on else None
        if on and self._captured is None:
            self._captured = torch.zeros(len(self.spec.schedule) + 1, self.spec.hidden_size, dtype=torch.float32,
                                         device=self.device)

    def captured_hidden(self) -> torch.Tensor:
        """[runs of the schedule + 1, hidden] float32 on the host: the residual of the captured token of the last
        step after the embedding (row 0) and after each layer run."""
        if self._captured is None:
            raise RuntimeError("nothing was captured: call set_capture_hidden(True) before the step")
        return self._captured.cpu()

    # ---------------------------------------------------------------------- step
    def step(self, entries: Sequence[StepEntry], n_prev: int = 0) -> Optional[torch.Tensor]:
        """Runs the entries as one batch; returns logits [wanted rows, vocab] fp32 on the device
        (a view of a scratch buffer, valid until the next step), or None if nothing is wanted.
        With ``n_prev`` > 0 a token -(r + 1), r < n_prev, is read on the device from ``sampled_ids[r]``."""
        graphable = self.cuda_graphs and self._capture_row is None and 0 < len(entries) <= self.graph_max_runs and \
            all(len(e.tokens) == 1 for e in entries)
        min_widths, ctx_bucket = None, None
        if graphable:
            # a graph is built for a bucket of context lengths: block tables are padded to the bucket's
            # width and the attention splits cover the bucket, so any shorter context fits
            bucket = self.graph_context_bucket
            longest = 1 + max(self.cache.get(e.request).tokens for e in entries)
            ctx_bucket = (longest + bucket - 1) // bucket * bucket
            min_widths = [max(1, ctx_bucket // self.cache.page_tokens) if g.paged else 1 for g in self.cache.groups]
        staging = []

        def alloc(n: int):
            host, event = self.workspace.pinned_ints(n)
            staging.append((host, event))
            return host.numpy(), host.data_ptr()

        packed = self._packer.pack(entries, self.cache, self.spec.vocab_size, self.spec.max_positions,
                           tile_keys=self.model.tile_requests(), min_widths=min_widths, alloc=alloc,
                                   n_prev=min(int(n_prev), self.sampled_ids.numel()))
        packed.staging = staging[0]
        return self.run_batch(packed, ctx_bucket)

    def run_batch(self, batch, graph_bucket: Optional[int] = None) -> Optional[torch.Tensor]:
        """Runs a laid-out step (a ``PackedStep``, or a ``StepBatch`` which is packed here)."""
        if batch.T > self.max_batch_tokens:
            raise BatchError(f"the step has {batch.T} tokens; the limit is {self.max_batch_tokens}")
        if graph_bucket is not None:
            logits = self._run_decode_graph(batch, graph_bucket)
        else:
            ctx = StepContext(batch, self.workspace, self.device, self.max_batch_tokens, err=self.err,
                              tile_sizes=self.model.tile_requests(), prev_ids=self.sampled_ids)
            if self._capture_row is not None:
                ctx.capture_hidden = (self._capture_row, self._captured)
            logits = self.model.forward(ctx, self.storage)
        lens = batch.context_len.tolist()
        for s, req in enumerate(batch.requests):
            self.cache.advance(req, lens[s])
        self.steps += 1
        return logits

    def _run_decode_graph(self, packed, ctx_bucket: int) -> Optional[torch.Tensor]:
        """A decode step through a captured graph.  The first step of a shape runs eagerly (it also
        allocates every buffer), the second is captured, later ones only upload the step's integers
        and replay."""
        key = (packed.S, packed.R, ctx_bucket, tuple(packed.widths))
        ctx = StepContext(packed, self.workspace, self.device, self.max_batch_tokens, err=self.err,
                          max_context=ctx_bucket, prev_ids=self.sampled_ids)          # uploads this step's integers
        entry = self._graphs.get(key)
        if (entry is not None and entry[1] == self.workspace.version and entry[3] == ctx.ints.data_ptr()
                and entry[5] == ops.scratch_version()):
            entry[0].replay()
            self.graph_replays += 1
            ops.add_launches(entry[4])
            return entry[2]
        if key not in self._graph_seen:
            self._graph_seen.add(key)
            return self.model.forward(ctx, self.storage)
        version, scratch_version = self.workspace.version, ops.scratch_version()
        n0 = ops.launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            cap = StepContext(packed, self.workspace, self.device, self.max_batch_tokens, err=self.err,
                              max_context=ctx_bucket, upload=False, prev_ids=self.sampled_ids)
            logits = self.model.forward(cap, self.storage)
        if (self.workspace.version != version or cap.ints.data_ptr() != ctx.ints.data_ptr()
                or ops.scratch_version() != scratch_version):
            # a buffer was (re)allocated while capturing: the graph holds stale pointers; run eagerly
            self._graph_seen.discard(key)
            return self.model.forward(ctx, self.storage)
        if len(self._graphs) > 64:
            self._graphs.clear()
        self._graphs[key] = (graph, version, logits, ctx.ints.data_ptr(), ops.launch_count() - n0, scratch_version)
        graph.replay()
        self.graph_replays += 1
        return logits

    @staticmethod
    def describe_error(code: int) -> str:
        what = [n for b, n in ((1, "a token id outside the vocabulary"), (2, "a page id outside the pool"),
                               (4, "a bounded wait ran out")) if code & b]
        return "a kernel reported: " + (", ".join(what) or f"error word {code}")

    def read_error(self) -> int:
        """The kernels' error word (synchronises)."""
        return int(self.err.item())

    def reset_after_error(self) -> None:
        """After a reported error: clears the error word and the split-K scratch, which an aborted product may
        have left non-zero (every later product relies on finding it zeroed)."""
        self.err.zero_()
        ops.zero_scratch(self.device)

    def check_device(self) -> None:
        """Raises if a kernel recorded an out-of-range index or a wait that ran out (synchronises)."""
        code = self.read_error()
        if code:
            self.reset_after_error()
            raise DeviceError(self.describe_error(code))
