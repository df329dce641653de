"""Qwen3 dense (``Qwen3ForCausalLM``): typed configuration from config.json.

Keys, defaults and checks follow the reference's reader (src/model/config.cpp:18-62):
required ``vocab_size``, ``hidden_size``, ``intermediate_size``, ``num_hidden_layers``,
``num_attention_heads``; ``num_key_value_heads`` defaults to the head count,
``head_dim`` to hidden/heads, ``rms_norm_eps`` 1e-6, ``rope_theta`` 10000,
``max_position_embeddings`` 4096, ``tie_word_embeddings`` false, ``attention_bias``
false; ``rope_scaling`` must be absent or null; heads must be a multiple of kv heads;
head_dim even and at most 256; EOS ids come from generation_config.json first.
Per-head q/k RMSNorm is on for this architecture (config.cpp:34) and uses
``rms_norm_eps`` (src/backend/cpu/cpu_backend.cpp:158-166).
"""
from __future__ import annotations

from dataclasses import dataclass, field, asdict
from typing import Mapping, Optional, Tuple

from .spec import (AttentionSpec, ConfigError, GatedMLPSpec, LayerSpec, ModelSpec,
                   RMSNormSpec, RotarySpec, default_schedule)
from .registry import register_architecture

_REQUIRED = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads")


def _int(config: Mapping, key: str, default=None) -> int:
    v = config.get(key, default)
    if v is None:
        raise ConfigError(f"config.json lacks the required key {key!r}")
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
        raise ConfigError(f"config.json: {key} must be an integer, got {v!r}")
    return int(v)


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    max_position_embeddings: int = 4096
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    hidden_act: str = "silu"
    initializer_range: float = 0.02
    eos_token_ids: Tuple[int, ...] = ()
    # config.json's use_sliding_window / sliding_window / max_window_layers: the first max_window_layers
    # layers see all keys, the layers after them only the last sliding_window (their own position included).
    # The reference has no such layers (it ignores the keys); here they are a second cache group.
    use_sliding_window: bool = False
    sliding_window: int = 0
    max_window_layers: int = 0

    architecture = "Qwen3ForCausalLM"
    model_type = "qwen3"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_json(cls, config: Mapping, generation_config: Optional[Mapping] = None) -> "Qwen3Config":
        for k in _REQUIRED:
            if config.get(k) is None:
                raise ConfigError(f"config.json lacks the required key {k!r}")
        heads = _int(config, "num_attention_heads")
        hidden = _int(config, "hidden_size")
        if heads <= 0:
            raise ConfigError("config.json has non-positive dimensions")
        kv_heads = _int(config, "num_key_value_heads", heads) if config.get("num_key_value_heads") is not None else heads
        head_dim = _int(config, "head_dim", hidden // heads) if config.get("head_dim") is not None else hidden // heads
        if config.get("rope_scaling") is not None:
            raise ConfigError("rope_scaling is not supported")
        use_window = bool(config.get("use_sliding_window", False))
        window = _int(config, "sliding_window", 0) if config.get("sliding_window") is not None else 0
        window_from = _int(config, "max_window_layers", 0) if config.get("max_window_layers") is not None else 0
        if use_window and window <= 0:
            raise ConfigError("use_sliding_window=true needs a positive sliding_window")
        act = config.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act {act!r} is not supported (silu only)")

        def eos(src):
            if not src:
                return ()
            v = src.get("eos_token_id")
            if v is None:
                return ()
            if isinstance(v, (list, tuple)):
                return tuple(int(x) for x in v)
            return (int(v),)

        eos_ids = eos(generation_config) or eos(config)
        out = cls(
            vocab_size=_int(config, "vocab_size"),
            hidden_size=hidden,
            intermediate_size=_int(config, "intermediate_size"),
            num_hidden_layers=_int(config, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=float(config.get("rms_norm_eps") if config.get("rms_norm_eps") is not None else 1e-6),
            rope_theta=float(config.get("rope_theta") if config.get("rope_theta") is not None else 10000.0),
            max_position_embeddings=_int(config, "max_position_embeddings", 4096)
            if config.get("max_position_embeddings") is not None else 4096,
            tie_word_embeddings=bool(config.get("tie_word_embeddings", False)),
            attention_bias=bool(config.get("attention_bias", False)),
            hidden_act=act,
            initializer_range=float(config.get("initializer_range") or 0.02),
            eos_token_ids=eos_ids,
            use_sliding_window=use_window,
            sliding_window=window if use_window else 0,
            max_window_layers=max(0, window_from) if use_window else 0,
        )
        out.validate()
        return out

    def validate(self) -> None:
        dims = (self.vocab_size, self.hidden_size, self.intermediate_size, self.num_hidden_layers,
                self.num_attention_heads, self.num_key_value_heads, self.head_dim, self.max_position_embeddings)
        if any(d <= 0 for d in dims):
            raise ConfigError("config.json has non-positive dimensions")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError("num_attention_heads must be a multiple of num_key_value_heads")
        if self.head_dim % 2 != 0 or self.head_dim > 256:
            raise ConfigError("head_dim must be even and at most 256")
        if not (self.rms_norm_eps > 0):
            raise ConfigError("rms_norm_eps must be positive")
        if not (self.rope_theta > 0):
            raise ConfigError("rope_theta must be positive")

    # ------------------------------------------------------------------ derived
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def parameters(self) -> int:
        """Parameter count (src/model/config.cpp:10-16)."""
        h = self.hidden_size
        attn = h * (self.q_dim + 2 * self.kv_dim) + self.q_dim * h
        mlp = 3 * h * self.intermediate_size
        norms = 2 * h + 2 * self.head_dim
        embed = self.vocab_size * h
        return self.num_hidden_layers * (attn + mlp + norms) + embed * (1 if self.tie_word_embeddings else 2) + h

    def kv_bytes_per_token(self, elem_bytes: int) -> int:
        return 2 * self.num_hidden_layers * self.kv_dim * elem_bytes

    def describe(self) -> str:
        return (f"qwen3 with {self.parameters() / 1e9:.2f}B parameters: {self.num_hidden_layers} layers, "
                f"d={self.hidden_size}, {self.num_attention_heads} heads ({self.num_key_value_heads} kv) x "
                f"{self.head_dim}, mlp {self.intermediate_size}, vocab {self.vocab_size}")

    def to_json(self) -> dict:
        """The config.json that reads back as this configuration."""
        d = {
            "architectures": [self.architecture],
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.attention_bias,
            "hidden_act": self.hidden_act,
            "initializer_range": self.initializer_range,
        }
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        if self.use_sliding_window:
            d.update(use_sliding_window=True, sliding_window=self.sliding_window, max_window_layers=self.max_window_layers)
        return d

    def layer_window(self, layer: int) -> int:
        """Keys a query of this layer sees (its own included); 0 = all."""
        return self.sliding_window if self.use_sliding_window and layer >= self.max_window_layers else 0

    # --------------------------------------------------------------- as a model
    def to_model_spec(self) -> ModelSpec:
        """Pre-norm decoder, L layers that differ at most in their window (cpu_backend.cpp:139-213), final
        norm, tied or untied head (cpu_backend.cpp:51-53)."""
        rope = RotarySpec(head_dim=self.head_dim, rotary_dim=self.head_dim, theta=self.rope_theta)

        def attn(layer: int) -> AttentionSpec:
            return AttentionSpec(hidden_size=self.hidden_size, num_heads=self.num_attention_heads,
                                 num_kv_heads=self.num_key_value_heads, head_dim=self.head_dim,
                                 qk_norm=True, qk_norm_eps=self.rms_norm_eps, bias=self.attention_bias,
                                 window=self.layer_window(layer), softmax_scale=None, position=rope)

        mlp = GatedMLPSpec(hidden_size=self.hidden_size, intermediate_size=self.intermediate_size,
                           activation=self.hidden_act)
        norm = RMSNormSpec(size=self.hidden_size, eps=self.rms_norm_eps)
        layers = tuple(
            LayerSpec.prenorm(mixer=attn(i), feed_forward=mlp, mixer_norm=norm, feed_forward_norm=norm,
                              mixer_prefix=f"model.layers.{i}.self_attn.", feed_forward_prefix=f"model.layers.{i}.mlp.",
                              mixer_norm_prefix=f"model.layers.{i}.input_layernorm.",
                              feed_forward_norm_prefix=f"model.layers.{i}.post_attention_layernorm.")
            for i in range(self.num_hidden_layers))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab_size, hidden_size=self.hidden_size,
            layers=layers, schedule=default_schedule(self.num_hidden_layers), final_norm=norm,
            final_norm_prefix="model.norm.",
            embedding_name="model.embed_tokens.weight", head_name="lm_head.weight",
            tie_embeddings=self.tie_word_embeddings, head_optional=True,
            max_positions=self.max_position_embeddings, eos_ids=self.eos_token_ids,
            init_std=self.initializer_range)


register_architecture(Qwen3Config.architecture, Qwen3Config, model_type=Qwen3Config.model_type)
