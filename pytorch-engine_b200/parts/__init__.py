"""Parts of a decoder: norms, position encodings, mixers, feed-forwards, block arrangements,
embedding and head, each registered under a kind and built from a ``PartSpec``."""
from . import registry, spec
from .registry import lookup, register, registered, unregister
from .spec import BlockSpec, CacheRequest, ModelPlan, PartSpec, RunStep, WeightDecl
from .runtime import Runtime
from . import norm, rope, attention, swiglu, embedding, block  # noqa: F401  (registers the built-in kinds)

__all__ = ["registry", "spec", "lookup", "register", "registered", "unregister", "BlockSpec", "CacheRequest",
           "ModelPlan", "PartSpec", "RunStep", "WeightDecl", "Runtime"]
