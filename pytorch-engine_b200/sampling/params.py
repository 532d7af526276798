"""Sampling options, with the reference's names, meanings and defaults
(``SamplingConfig``, pygguf_engine/engine.py:28-45; order of the filters 82-134)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class SamplingParams:
    max_tokens: int = 512            # new-token limit, clamped to the context (engine.py:528)
    temperature: float = 0.7         # <= 1e-5: greedy argmax (engine.py:99-100, 146-147)
    top_p: float = 0.95              # 1.0 = off (engine.py:116-124)
    top_k: int = 40                  # 0 = off (engine.py:104-108)
    min_p: float = 0.05              # 0.0 = off (engine.py:112-114)
    repetition_penalty: float = 1.0  # on the unique ids of the last 256 tokens (engine.py:92-97)
    stop_token_ids: List[int] = field(default_factory=list)  # added to the configuration's eos ids
    seed: Optional[int] = None       # None: a fresh seed per call

    def validate(self) -> None:
        if self.max_tokens < 1:
            raise ValueError(f"max_tokens must be >= 1, got {self.max_tokens}")
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, got {self.top_k}")
        if not 0.0 <= self.min_p <= 1.0:
            raise ValueError(f"min_p must be in [0, 1], got {self.min_p}")
        if self.repetition_penalty <= 0:
            raise ValueError(f"repetition_penalty must be > 0, got {self.repetition_penalty}")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 1e-5

    @classmethod
    def greedy_params(cls, max_tokens: int = 512, **kw) -> "SamplingParams":
        return cls(max_tokens=max_tokens, temperature=0.0, top_p=1.0, top_k=0, min_p=0.0, **kw)
