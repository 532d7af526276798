"""A small, whole, single-GPU generation library for NVIDIA B200 (sm_100a): typed configuration and
registry, weights by name, decoder parts, a paged cache, one step function, a generation loop,
sampling, and hand-written CUDA kernels.  One architecture is built in: the Qwen3 dense decoder."""
from . import config, parts, cache, weights, kernels, sampling, architectures, engine
from .config import ConfigError, Qwen3Config, load_config, preset, register_architecture
from .engine import Engine, GenerationResult, StepEntry, StreamChunk
from .sampling import SamplingParams
from .weights import WeightError, load_weights, write_random_model

__all__ = ["config", "parts", "cache", "weights", "kernels", "sampling", "architectures", "engine", "ConfigError",
           "Qwen3Config", "load_config", "preset", "register_architecture", "Engine", "GenerationResult", "StepEntry",
           "StreamChunk", "SamplingParams", "WeightError", "load_weights", "write_random_model"]
