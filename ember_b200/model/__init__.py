"""Model assembly from a ModelSpec."""
from .causal_lm import CausalLM, build_model

__all__ = ["CausalLM", "build_model"]
