"""The Python entry point: a model folder (or a configuration and a seed) to generated tokens.

Usage follows the reference's ``PyGGUFEngine(path, ...)`` then ``.generate(prompt_or_ids, sampling)``
(pygguf_engine/engine.py:259-291, 937-950), with its option names where it has them
(``max_context_len``, ``enable_cuda_graph``) and batches where it has one sequence:

    engine = Engine("model_dir", dtype="bfloat16", max_context_len=4096)
    result = engine.generate([1, 2, 3], SamplingParams(max_tokens=16, temperature=0.0))
    results = engine.generate([[1, 2, 3], [4, 5]], SamplingParams(...))     # a batch
    for chunk in engine.stream_tokens([[1, 2, 3]]): ...

It runs on one CUDA device and refuses to start without the package's CUDA library.
"""
from __future__ import annotations

import time
from typing import Dict, Iterator, List, Optional, Sequence, Union

import torch

from .. import architectures  # noqa: F401  (registers the built-in architectures)
from ..cache import PAGE_TOKENS, PagedCache, pages_for
from ..config.base import ModelConfig
from ..config.registry import architecture, load_config
from ..kernels import KernelError, library
from ..parts.runtime import Runtime
from ..sampling import Sampler, SamplingParams
from ..weights import load_weights, random_weights
from .batch import StepEntry
from .generate import GenerationLoop, GenerationResult, StreamChunk
from .model import DecoderModel
from .runner import ModelRunner

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def resolve_dtype(dtype: Union[str, torch.dtype]) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, got {dtype}")
        return dtype
    if dtype not in _DTYPES:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got {dtype!r}")
    return _DTYPES[dtype]


class _LoopBackend:
    """What the generation loop drives.  A step is not followed by a read of the status word of its
    own: the sampler's single device-to-host copy brings the tokens and the status word together."""

    def __init__(self, engine: "Engine") -> None:
        self.engine = engine
        self.alloc_slot = engine.alloc_slot
        self.free_slot = engine.free_slot
        self.free_pages = engine.free_pages
        self.sample = engine.sample

    def step(self, entries):
        return self.engine.runner.step(entries, check=False)

    def launch_decode(self, slots, tokens, params, seed, requests, steps):
        """Launch one decode step and its draw without waiting.  ``tokens``: the input tokens as a list,
        or None to take the tokens that the previous launch drew (still on the device).  Returns a handle
        with ``result() -> tokens``, or None if this cannot be done without the host in between."""
        eng = self.engine
        if tokens is None:
            if not eng.runner.can_step_from_device_tokens(len(slots)):
                return None
            logits = eng.runner.step_from_device_tokens(slots, eng.runtime.token_area)
        else:
            logits = eng.runner.step([StepEntry(s, (t,), (0,)) for s, t in zip(slots, tokens)], check=False)
        return eng.sampler.sample_async(logits, params, seed, requests, steps)


class Engine:
    def __init__(self, model_path: Optional[str] = None, *, dtype: Union[str, torch.dtype] = "bfloat16",
                 max_context_len: Optional[int] = None, max_cache_tokens: Optional[int] = None, max_batch: int = 64,
                 max_slots: Optional[int] = None, max_step_tokens: Optional[int] = 65536,
                 enable_cuda_graph: bool = True, device: str = "cuda:0",
                 config: Optional[ModelConfig] = None, weights: Optional[Dict[str, torch.Tensor]] = None,
                 verbose: bool = False) -> None:
        """``model_path``: a folder with config.json and model.safetensors.  ``max_context_len``: the
        longest sequence (default: the configuration's ``max_position_embeddings``).
        ``max_cache_tokens``: how many tokens all live sequences may hold together, each rounded up
        to 64 (default: ``max_batch`` sequences of full length, capped by free memory).
        ``max_step_tokens``: the most prompt tokens that generation feeds in one step (None: no limit); the
        buffers of a step, beside the cache, grow with its tokens (about 100 KB per token at the 8B shape)."""
        t0 = time.perf_counter()
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device is visible: this engine runs on a B200 (sm_100a) only and has no CPU path")
        library()  # build or load the CUDA library now; raises if that is impossible
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.dtype = resolve_dtype(dtype)
        if config is None:
            if model_path is None:
                raise ValueError("give a model folder, or a configuration with weights")
            config = load_config(model_path)
        self.config = config
        arch = architecture(config.architecture)
        self.plan = arch.plan(config)
        self.runtime = Runtime(self.device, self.dtype)
        if weights is None:
            weights = load_weights(model_path, self.plan, device=self.device, dtype=self.dtype)
        self.model = DecoderModel(self.plan, weights, self.runtime)
        del weights
        self.max_context_len = int(max_context_len or config.max_positions)
        if self.max_context_len > config.max_positions:
            raise ValueError(f"max_context_len {self.max_context_len} exceeds the model's max_position_embeddings "
                             f"{config.max_positions}")
        self.max_batch = int(max_batch)
        if max_cache_tokens is None:
            max_cache_tokens = self.default_cache_tokens(self.max_batch, self.max_context_len,
                                                         self.model.cache_requests(), self.dtype, self.device)
        self.max_cache_tokens = int(max_cache_tokens)
        if max_slots is None:
            max_slots = max(self.max_batch, min(pages_for(self.max_cache_tokens), 4096))
        self.cache = PagedCache(self.model.cache_requests(), max_tokens=self.max_cache_tokens, max_slots=max_slots,
                                max_seq_len=self.max_context_len, dtype=self.dtype, device=self.device)
        self.runner = ModelRunner(self.model, self.cache, cuda_graphs=enable_cuda_graph)
        self.sampler = Sampler(self.device, self.runtime)
        self.loop = GenerationLoop(_LoopBackend(self), max_context=self.max_context_len, max_batch=self.max_batch,
                                   eos_token_ids=config.stop_token_ids, bos_token_id=config.bos_token,
                                   max_step_tokens=max_step_tokens)
        self.load_time_s = time.perf_counter() - t0
        if verbose:
            rep = self.memory_report()
            print(f"[pytorch-engine_b200] {config.architecture} | dtype={self.dtype} | ctx={self.max_context_len} | "
                  f"weights={rep['weights_mib']} MiB | cache={rep['cache_mib']} MiB | load {self.load_time_s:.1f} s")

    # ---- constructors ------------------------------------------------------------------------
    @classmethod
    def from_pretrained(cls, model_path: str, **kw) -> "Engine":
        return cls(model_path, **kw)

    @staticmethod
    def default_cache_tokens(max_batch: int, max_context_len: int, requests, dtype, device, free_bytes=None) -> int:
        """``max_batch`` sequences of full length, but no more tokens than fit in four fifths of the
        device memory that is free now (whole pages; at least one page)."""
        want = max_batch * pages_for(max_context_len) * PAGE_TOKENS
        per_token = sum(2 * r.kv_heads * r.head_dim for r in requests.values() if r is not None and r.kind == "kv")
        per_token *= torch.empty((), dtype=dtype).element_size()
        if per_token == 0:
            return want
        if free_bytes is None:
            free_bytes = torch.cuda.mem_get_info(device)[0] if torch.device(device).type == "cuda" else 1 << 62
        fit = int(free_bytes * 0.8) // per_token // PAGE_TOKENS * PAGE_TOKENS
        return max(PAGE_TOKENS, min(want, fit))

    @classmethod
    def from_random(cls, config: ModelConfig, seed: int = 0, **kw) -> "Engine":
        """Random weights made directly on the device from ``seed`` (no files)."""
        device = kw.get("device", "cuda:0")
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device is visible: this engine runs on a B200 (sm_100a) only and has no CPU path")
        plan = architecture(config.architecture).plan(config)
        weights = random_weights(plan, seed, device=device)
        return cls(None, config=config, weights=weights, **kw)

    # ---- backend of the generation loop --------------------------------------------------------
    def alloc_slot(self) -> int:
        return self.runner.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self.runner.free_slot(slot)

    def free_pages(self) -> int:
        return self.cache.free_pages()

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """The step function (see ``engine/runner.py``): float32 logits at the wanted positions."""
        return self.runner.step(entries)

    def sample(self, logits, params, seed, requests, steps, recent=None) -> List[int]:
        return self.sampler.sample(logits, params, seed, requests, steps, recent)

    # ---- generation ----------------------------------------------------------------------------
    @staticmethod
    def _as_batch(prompt_or_prompts):
        if len(prompt_or_prompts) > 0 and isinstance(prompt_or_prompts[0], (list, tuple)):
            return [list(p) for p in prompt_or_prompts], True
        return [list(prompt_or_prompts)], False

    @torch.no_grad()
    def generate(self, prompt_or_ids, sampling: Optional[SamplingParams] = None):
        """Token ids in, ``GenerationResult`` out; a list of prompts gives a list of results."""
        prompts, many = self._as_batch(prompt_or_ids)
        results = self.loop.generate(prompts, sampling)
        return results if many else results[0]

    def stream_tokens(self, prompt_or_ids, sampling: Optional[SamplingParams] = None) -> Iterator[StreamChunk]:
        prompts, _ = self._as_batch(prompt_or_ids)
        # no_grad rather than inference_mode: buffers made here are also written by later calls of
        # step(), which may come from outside any such context.  It is entered for each advance of the
        # loop and left before the chunk is handed out, so the caller's own code between two chunks
        # runs in the caller's grad mode.
        chunks = self.loop.stream(prompts, sampling)
        try:
            while True:
                with torch.no_grad():
                    try:
                        chunk = next(chunks)
                    except StopIteration:
                        return
                yield chunk
        finally:
            chunks.close()

    # ---- reports -----------------------------------------------------------------------------
    def memory_report(self) -> Dict[str, float]:
        """Bytes held, in MiB (the reference's ``vram_report``, pygguf_engine/engine.py:471-508)."""
        mib = 1024.0 ** 2
        return {
            "weights_mib": round(self.model.weight_bytes() / mib, 2),
            "cache_mib": round(self.cache.nbytes() / mib, 2),
            "workspace_mib": round(self.runner.workspace_bytes() / mib, 2),
            "allocated_mib": round(torch.cuda.memory_allocated(self.device) / mib, 2),
        }
