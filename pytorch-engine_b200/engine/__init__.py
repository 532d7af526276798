"""The step function, the generation loop above it, and the Python entry point."""
from .batch import BufferPool, StepContext, StepEntry
from .generate import GenerationLoop, GenerationResult, StreamChunk
from .model import DecoderModel
from .runner import ModelRunner
from .engine import Engine, resolve_dtype
from . import replay
from .replay import TraceReplayer

__all__ = ["BufferPool", "StepContext", "StepEntry", "GenerationLoop", "GenerationResult", "StreamChunk",
           "DecoderModel", "ModelRunner", "Engine", "resolve_dtype", "replay", "TraceReplayer"]
