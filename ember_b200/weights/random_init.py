"""Random-weights mode: a model folder (config.json, model.safetensors) from a configuration
and a seed.

Every tensor a model declares is filled from its own generator, seeded by the seed and the
tensor's name, so a tensor's values do not depend on which other tensors exist: matrices
N(0, std), norm weights 1 + N(0, norm_std), biases N(0, std).  The reference has no such mode
(its tests need downloaded models); this one is what tests and the benchmark run on.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Iterator, Optional, Tuple

import torch

from ..config.spec import ModelSpec
from .safetensors_io import save_file


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


class RandomSource:
    """The tensors of the random-weights mode as a source a ``WeightStore`` reads from: each tensor is made when
    it is asked for and not kept, so a large model never exists twice (once as made, once as loaded)."""

    def __init__(self, spec: ModelSpec, seed: int, dtype: torch.dtype = torch.bfloat16, std: Optional[float] = None,
                 norm_std: Optional[float] = None, device: str = "cpu"):
        from ..model.causal_lm import CausalLM
        self.seed, self._dtype, self.device = seed, dtype, device
        self.std = spec.init_std if std is None else std
        self.norm_std = spec.init_norm_std if norm_std is None else norm_std
        self._decls = {d.name: d for d in CausalLM(spec).weight_decls()}

    def names(self):
        return list(self._decls)

    def has(self, name: str) -> bool:
        return name in self._decls

    def shape(self, name: str):
        return tuple(self._decls[name].shape)

    def dtype(self, name: str) -> torch.dtype:
        return self._dtype

    def get(self, name: str) -> torch.Tensor:
        d = self._decls[name]
        g = torch.Generator(device=self.device)
        g.manual_seed(_tensor_seed(self.seed, d.name))
        t = torch.empty(d.shape, dtype=torch.float32, device=self.device)
        if d.init == "norm":
            t.normal_(0.0, self.norm_std, generator=g).add_(1.0)
        else:                                   # matrices, and biases ("zeros" names what a trained model often has)
            t.normal_(0.0, self.std, generator=g)
        return t.to(self._dtype)


def random_tensors(spec: ModelSpec, seed: int, dtype: torch.dtype = torch.bfloat16,
                   std: Optional[float] = None, norm_std: Optional[float] = None,
                   device: str = "cpu") -> Iterator[Tuple[str, torch.Tensor]]:
    """Yields (name, tensor) for every tensor the model declares (optional ones included unless tied)."""
    src = RandomSource(spec, seed, dtype, std, norm_std, device)
    for name in src.names():
        yield name, src.get(name)


def write_model_dir(config, out_dir: str, seed: int, dtype: torch.dtype = torch.bfloat16,
                    std: Optional[float] = None, norm_std: Optional[float] = None) -> str:
    """Writes ``out_dir/config.json`` and ``out_dir/model.safetensors`` for ``config`` (an
    architecture's configuration object with ``to_json`` and ``to_model_spec``)."""
    os.makedirs(out_dir, exist_ok=True)
    spec = config.to_model_spec()
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_json(), f, indent=2)
    tensors: Dict[str, torch.Tensor] = dict(random_tensors(spec, seed, dtype, std, norm_std))
    save_file(tensors, os.path.join(out_dir, "model.safetensors"),
              metadata={"format": "pt", "seed": str(seed), "generator": "ember_b200.random_init"})
    return out_dir
