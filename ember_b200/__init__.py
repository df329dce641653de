"""ember_b200: a small, whole LLM inference engine for one NVIDIA B200.

From a model folder (config.json + safetensors) or a seeded random-weights mode to generated
tokens: typed configuration and registry, named weight loading, parts (norm, position
encoding, mixer, feed-forward) arranged into blocks by data, a paged cache manager, one step
function over mixed batches, a continuous-batching scheduler, device sampling, and
hand-written sm_100a kernels in bfloat16 with a true float32 path beside them.
"""
from .sampling.params import SamplingParams
from .engine.batch import StepEntry
from .engine.scheduler import Request

__version__ = "0.1.0"


def load(*args, **kw):
    from .api import load as _load
    return _load(*args, **kw)


def load_random(*args, **kw):
    from .api import load_random as _load_random
    return _load_random(*args, **kw)


__all__ = ["SamplingParams", "StepEntry", "Request", "load", "load_random", "__version__"]
