"""The tests' own tiny Qwen3 configurations.  They differ in every size and option: layers,
width, heads and groups, head size, projection width vs model width, feed-forward width,
vocabulary (one a power of two, one not), rope theta, norm eps, tied vs untied head, initial
scales, position limit, biases, a sliding window on some of the layers."""
from __future__ import annotations

import numpy as np

from ember_b200.config import Qwen3Config

TINY = {
    "a": dict(seed=11, std=0.02, norm_std=0.05,
              json=dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=512, hidden_size=64,
                        intermediate_size=192, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                        head_dim=16, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                        max_position_embeddings=128, attention_bias=False)),
    "b": dict(seed=23, std=0.03, norm_std=0.1,
              json=dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=1000, hidden_size=96,
                        intermediate_size=256, num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=1,
                        head_dim=32, rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
                        max_position_embeddings=256, attention_bias=False)),
    # two more shapes that reach the tensor-core attention kernels in bfloat16: head size 128 with a
    # group of 2 (tcgen05 prompt kernel + key-split decode kernel) and head size 64 with a group of 3
    "c": dict(seed=31, std=0.04, norm_std=0.08,
              json=dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=777, hidden_size=256,
                        intermediate_size=328, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                        head_dim=128, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                        max_position_embeddings=512, attention_bias=False)),
    "d": dict(seed=37, std=0.04, norm_std=0.08,
              json=dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=640, hidden_size=136,
                        intermediate_size=200, num_hidden_layers=2, num_attention_heads=3, num_key_value_heads=1,
                        head_dim=64, rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
                        max_position_embeddings=512, attention_bias=False)),
    # sizes the tensor-core kernels refuse (a width of 100 breaks the 16-byte row rule of TMA, head size 48
    # is no multiple of 32), q/k/v biases, as many key heads as query heads: the general kernels in bfloat16
    "e": dict(seed=41, std=0.05, norm_std=0.1,
              json=dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=333, hidden_size=100,
                        intermediate_size=150, num_hidden_layers=2, num_attention_heads=5, num_key_value_heads=5,
                        head_dim=48, rope_theta=50000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                        max_position_embeddings=300, attention_bias=True)),
    # layers that differ: the first sees all keys, the two after it a window of 24 (two cache groups; window pages
    # are given back while a request runs); head size 64 with a group of 2
    "f": dict(seed=43, std=0.05, norm_std=0.1,
              json=dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=450, hidden_size=128,
                        intermediate_size=176, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                        head_dim=64, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                        max_position_embeddings=400, attention_bias=False, use_sliding_window=True, sliding_window=24,
                        max_window_layers=1)),
}
GOLDEN_CONFIGS = ("a", "b")          # the ones the reference's CPU backend was run on


def tiny_config(name: str) -> Qwen3Config:
    return Qwen3Config.from_json(TINY[name]["json"])


def tiny_prompts(name: str):
    rng = np.random.default_rng(1234 + ord(name))
    vocab = TINY[name]["json"]["vocab_size"]
    lengths = (5, 17, 33) if name == "a" else (1, 31, 64, 100)          # "b", "c", "d": the longer set
    return [rng.integers(0, vocab, size=n).tolist() for n in lengths]
