"""A small, whole inference engine for the dense Llama decoder on one B200.

From a model folder (config.json + model.safetensors) or a seeded random
configuration to generated tokens: typed configuration and an architecture
registry, weights by tensor name, layers put together from parts, a paged
key/value cache, one step function over mixed batches, a scheduler, sampling,
and hand-written CUDA kernels for sm_100a.  Importing the package does not
touch the GPU; ``Engine`` does.
"""
__version__ = "0.1.0"

from .config.llama import ConfigError, LlamaConfig, RopeScaling  # noqa: F401
from .config.registry import known_architectures, register_architecture, resolve  # noqa: F401


def __getattr__(name):
    # heavier pieces are imported on first use
    if name in ("Engine", "EngineParams", "StepEntry", "random_engine"):
        from .engine import engine as _e
        return getattr(_e, name)
    if name in ("Runner", "SamplingParams", "GenerationResult"):
        from .engine import runner as _r
        return getattr(_r, name)
    raise AttributeError(name)
