"""Typed description of a model as data: parts, layers, and the order they run in.

An architecture's configuration class (for instance ``Qwen3Config``) turns the keys
of its ``config.json`` into a ``ModelSpec``.  Everything below the configuration
(weights, parts, cache manager, step function) reads only the ``ModelSpec``; no
size or constant of a model is written anywhere else.

A part spec is a frozen dataclass with a class attribute ``kind``; the part
registry (``ember_b200.parts.registry``) maps ``(family, kind)`` to the class that
implements it.  A test or a user can define a new spec + part pair and register it
without touching the framework's files.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import ClassVar, Optional, Tuple


class ConfigError(ValueError):
    """A configuration that cannot be built (missing key, bad value, unsupported option)."""


@dataclass(frozen=True)
class PartSpec:
    """Base of all part specs.  ``kind`` selects the implementation in the registry."""

    kind: ClassVar[str] = ""


# ----------------------------------------------------------------------------- norms
@dataclass(frozen=True)
class RMSNormSpec(PartSpec):
    """out = weight * (x * rsqrt(mean(x^2) + eps)); plain weight (not 1 + weight)."""

    kind: ClassVar[str] = "rmsnorm"
    size: int = 0
    eps: float = 1e-6


# ---------------------------------------------------------------- position encodings
@dataclass(frozen=True)
class RotarySpec(PartSpec):
    """Rotate-half rotary embedding over the first ``rotary_dim`` elements of a head."""

    kind: ClassVar[str] = "rope"
    head_dim: int = 0
    rotary_dim: int = 0          # == head_dim for a full rotation
    theta: float = 10000.0


@dataclass(frozen=True)
class NoPositionSpec(PartSpec):
    kind: ClassVar[str] = "none"


# ---------------------------------------------------------------------------- mixers
@dataclass(frozen=True)
class AttentionSpec(PartSpec):
    """Grouped-query causal attention over a paged key/value cache."""

    kind: ClassVar[str] = "attention"
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    qk_norm: bool = False         # RMSNorm on each query/key head before the rotation
    qk_norm_eps: float = 1e-6
    bias: bool = False            # biases on the q/k/v projections
    window: int = 0               # 0 = all keys; w > 0 = the last w keys (self included)
    softmax_scale: Optional[float] = None   # None = 1/sqrt(head_dim)
    position: PartSpec = field(default_factory=NoPositionSpec)

    @property
    def q_dim(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def group(self) -> int:
        return self.num_heads // self.num_kv_heads


# --------------------------------------------------------------------- feed-forwards
@dataclass(frozen=True)
class GatedMLPSpec(PartSpec):
    """down( act(gate(x)) * up(x) ), no biases."""

    kind: ClassVar[str] = "gated_mlp"
    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "silu"


# ---------------------------------------------------------------------------- layers
@dataclass(frozen=True)
class LayerSpec:
    """One block: the name of its arrangement (a registered class) and the parts that arrangement puts around the
    residual stream, each under a *role*: ``(role, part spec, weight-name prefix)``.  Which roles exist, which
    family each belongs to and in what order they run is the arrangement's business ("prenorm" knows
    ``mixer_norm``, ``mixer``, ``feed_forward_norm``, ``feed_forward``); a block with four norms, with two mixers
    or without a feed-forward is another arrangement over another set of roles, not another ``LayerSpec``."""

    arrangement: str = "prenorm"
    parts: Tuple[Tuple[str, PartSpec, str], ...] = ()

    def __post_init__(self):
        roles = [r for r, _, _ in self.parts]
        if len(set(roles)) != len(roles):
            raise ConfigError(f"a layer names a role twice: {roles}")

    def roles(self) -> Tuple[str, ...]:
        return tuple(r for r, _, _ in self.parts)

    def part(self, role: str) -> Tuple[PartSpec, str]:
        for r, spec, prefix in self.parts:
            if r == role:
                return spec, prefix
        raise ConfigError(f"the layer has no part in the role {role!r} (it has: {', '.join(self.roles()) or 'none'})")

    @classmethod
    def prenorm(cls, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec, feed_forward_norm: PartSpec,
                mixer_prefix: str, feed_forward_prefix: str, mixer_norm_prefix: str,
                feed_forward_norm_prefix: str) -> "LayerSpec":
        """h += mixer(norm(h)); h += feed_forward(norm(h)): prefixes are, for instance, "model.layers.3.self_attn.",
        "model.layers.3.mlp.", "model.layers.3.input_layernorm.", "model.layers.3.post_attention_layernorm."."""
        return cls("prenorm", (("mixer_norm", mixer_norm, mixer_norm_prefix), ("mixer", mixer, mixer_prefix),
                               ("feed_forward_norm", feed_forward_norm, feed_forward_norm_prefix),
                               ("feed_forward", feed_forward, feed_forward_prefix)))


@dataclass(frozen=True)
class ScheduleEntry:
    """One position in the run order.  ``layer`` indexes ``ModelSpec.layers``; a layer
    may appear more than once.  ``cache_of`` names the layer whose cache this run
    reads and writes; -1 means its own."""

    layer: int
    cache_of: int = -1


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    final_norm_prefix: str = "model.norm."
    embedding_name: str = "model.embed_tokens.weight"
    head_name: str = "lm_head.weight"
    tie_embeddings: bool = False
    head_optional: bool = True            # untied but absent in the file => use the embedding
    max_positions: int = 4096
    eos_ids: Tuple[int, ...] = ()
    init_std: float = 0.02                # random-weights mode: std of linear weights
    init_norm_std: float = 0.05           # random-weights mode: norm weights are 1 + N(0, this)
    # a position encoding that acts on the embedded tokens (learned or sinusoidal tables); rotary ones
    # belong to their mixer's spec instead
    embedding_position: PartSpec = field(default_factory=NoPositionSpec)
    embedding_position_prefix: str = "model.embed_positions."
    # h = embedding_multiplier * table[token] and logits = logit_scale * (norm(h) . head^T): 1.0 for Qwen3; other
    # decoders scale the embedded tokens by sqrt(hidden) or the logits by a constant
    embedding_multiplier: float = 1.0
    logit_scale: float = 1.0

    def __post_init__(self):
        n = len(self.layers)
        if n == 0:
            raise ConfigError("a model needs at least one layer")
        if not self.schedule:
            raise ConfigError("the layer schedule is empty")
        for e in self.schedule:
            if not (0 <= e.layer < n):
                raise ConfigError(f"schedule names layer {e.layer}; the model has {n}")
            if not (-1 <= e.cache_of < n):
                raise ConfigError(f"schedule entry reads the cache of layer {e.cache_of}; the model has {n}")


def default_schedule(n_layers: int) -> Tuple[ScheduleEntry, ...]:
    return tuple(ScheduleEntry(i) for i in range(n_layers))
