"""The Python entry point: a model folder (or a configuration and a seed) to generated tokens.

    import ember_b200
    llm = ember_b200.load("path/to/model", dtype="bfloat16")
    ids = llm.generate([1, 2, 3], max_tokens=16)                       # greedy by default
    ids = llm.generate([[1, 2, 3], [4, 5]], sampling=ember_b200.SamplingParams(temperature=0.7, top_k=20))

Option names and meanings are the reference's (src/backend/backend.hpp:39-53,
src/engine/engine.hpp:77-84, tools/cli_args.hpp:57-88) where it has them.
"""
from __future__ import annotations

import os
import tempfile
from typing import List, Optional, Sequence, Union

import torch

from .config.registry import load_config
from .engine.engine import Engine
from .engine.runner import ModelRunner
from .sampling.params import SamplingParams
from .weights.loader import WeightStore
from .weights.random_init import RandomSource


class LLM:
    """A loaded model with its engine."""

    def __init__(self, runner: ModelRunner, max_prefill_chunk: int = 2048, max_context: Optional[int] = None):
        self.runner = runner
        self.engine = Engine(runner, max_prefill_chunk=max_prefill_chunk, max_context=max_context)

    @property
    def spec(self):
        return self.runner.spec

    def generate(self, prompts, sampling: Optional[SamplingParams] = None, max_tokens: int = 256,
                 ignore_eos: bool = False, stop_tokens: Sequence[int] = ()):
        """Token ids in (one prompt or a list of prompts), generated token ids out (host lists)."""
        return self.engine.generate(prompts, sampling=sampling, max_tokens=max_tokens, ignore_eos=ignore_eos,
                                    stop_tokens=stop_tokens)

    def step(self, entries):
        """The step function itself: ``[StepEntry(request, tokens, want)] -> logits`` (device, fp32)."""
        return self.runner.step(entries)

    @property
    def stats(self):
        return self.engine.stats


def load(model: str, dtype: str = "bfloat16", device: str = "cuda:0", kv_cache_tokens: int = 0,
         max_batch_tokens: int = 2048, max_seqs: int = 64, prefill_chunk: int = 2048,
         max_context: Optional[int] = None, page_tokens: int = 64, cuda_graphs: bool = True,
         gpu_memory: float = 0.92, kv_cache_mib: int = 0, strict_weights: bool = False) -> LLM:
    """Loads a model folder (config.json + safetensors).  The cache holds ``kv_cache_tokens`` tokens if given,
    else ``kv_cache_mib`` MiB if given, else what fits once the weights are on the device when ``gpu_memory`` of
    the device's memory may be used (the reference's --gpu-memory / --kv-cache-mib / --kv-cache-tokens,
    tools/cli_args.hpp:57-88; src/backend/cuda/cuda_backend.cu:757-780), and never more than ``max_seqs`` requests
    of ``max_context`` tokens could fill."""
    cfg = load_config(model)
    spec = cfg.to_model_spec()
    runner = ModelRunner(spec, WeightStore.from_dir(model, strict=strict_weights), dtype=dtype, device=device,
                         capacity_tokens=kv_cache_tokens, max_batch_tokens=max_batch_tokens,
                         max_requests=max_seqs, page_tokens=page_tokens, cuda_graphs=cuda_graphs,
                         memory_fraction=gpu_memory, cache_bytes=int(kv_cache_mib) << 20, max_context=max_context)
    return LLM(runner, max_prefill_chunk=prefill_chunk, max_context=max_context)


def load_random(config, seed: int = 0, dtype: str = "bfloat16", device: str = "cuda:0", kv_cache_tokens: int = 0,
                max_batch_tokens: int = 2048, max_seqs: int = 64, prefill_chunk: int = 2048,
                max_context: Optional[int] = None, page_tokens: int = 64, cuda_graphs: bool = True,
                weight_dtype=torch.bfloat16, std: Optional[float] = None, norm_std: Optional[float] = None,
                gpu_memory: float = 0.92, kv_cache_mib: int = 0) -> LLM:
    """Random-weights mode without a folder: the tensors are made from ``seed`` in memory
    (on the device when it is a CUDA device) and loaded as if they came from a file."""
    spec = config.to_model_spec()
    gen_device = device if torch.cuda.is_available() else "cpu"
    # tensors are made one at a time as the parts take them: a 65 GB model is never held twice
    store = WeightStore(RandomSource(spec, seed, weight_dtype, std, norm_std, device=gen_device),
                        description=f"random weights (seed {seed})")
    runner = ModelRunner(spec, store, dtype=dtype, device=device, capacity_tokens=kv_cache_tokens,
                         max_batch_tokens=max_batch_tokens, max_requests=max_seqs, page_tokens=page_tokens,
                         cuda_graphs=cuda_graphs, memory_fraction=gpu_memory, cache_bytes=int(kv_cache_mib) << 20,
                         max_context=max_context)
    return LLM(runner, max_prefill_chunk=prefill_chunk, max_context=max_context)
