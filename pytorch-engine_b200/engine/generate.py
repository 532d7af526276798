"""The generation loop above the step function.

Requests are taken in order, as many at a time as the batch limit and the cache allow; the
prompts of a batch (unequal lengths) go through one step, then every live sequence gets one token
per step; a sequence that draws a stop token or reaches its limit leaves the batch at once and
gives its slot back while the others go on; when a batch is finished the next one starts, until
no request is left.

Rules kept from the reference (pygguf_engine/engine.py): an empty prompt becomes ``[bos or 0]``
(525-526); the new-token limit is ``max(1, min(max_tokens, context - prompt length))`` (528); stop
ids are the configuration's eos ids plus the request's (529); the first token comes from the last
prompt row (637); a stop token ends the sequence and is not part of the output (638-651, 862-867);
the finish reason is "stop" or "length" (887-893); the newest token enters the cache in the next
step (685).

The loop decides; it does not compute.  ``backend`` supplies ``alloc_slot()``, ``free_slot(slot)``,
``free_pages()``, ``step(entries) -> logits`` and ``sample(logits, params, seed, requests, steps,
recent) -> tokens``, so the decisions can be tested without a GPU.  A backend may also offer
``launch_decode(slots, tokens_or_None, params, seed, requests, steps) -> handle`` (``handle.result()``
gives the drawn tokens): the loop then keeps one decode step queued ahead of the one whose tokens it
is reading, so the device never waits for the host between steps.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Iterator, List, Optional, Sequence, Tuple

from ..cache.paged import PAGE_TOKENS, pages_for
from ..sampling.params import SamplingParams
from .batch import StepEntry


@dataclass
class GenerationResult:
    """What one request produced (field names follow the reference's ``GenerationResult``,
    pygguf_engine/engine.py:48-71; ``text`` has no counterpart here: tokens in, tokens out)."""

    token_ids: List[int]
    prompt_tokens: int
    completion_tokens: int
    finish_reason: str  # "stop" | "length"
    prefill_time_s: float = 0.0
    decode_time_s: float = 0.0

    @property
    def prompt_tok_per_s(self) -> float:
        return max(1, self.prompt_tokens) / max(self.prefill_time_s, 1e-6)

    @property
    def decode_tok_per_s(self) -> float:
        return self.completion_tokens / max(self.decode_time_s, 1e-6)


@dataclass
class StreamChunk:
    """One new token of one request (``request`` indexes the prompts given to ``stream``)."""

    request: int
    token_id: int
    finish_reason: Optional[str] = None
    stats: Optional[GenerationResult] = None


@dataclass
class _Live:
    request: int
    slot: int
    prompt: List[int]
    max_new: int
    generated: List[int] = field(default_factory=list)


class GenerationLoop:
    def __init__(self, backend, *, max_context: int, max_batch: int, eos_token_ids: Sequence[int] = (),
                 bos_token_id: int = 0, max_step_tokens: Optional[int] = None) -> None:
        """``max_step_tokens``: the most prompt tokens one step brings (None: no limit).  A batch whose
        prompts hold more goes through several steps, a prompt longer than that in pieces: what a step
        needs beside the cache grows with its tokens."""
        self.backend = backend
        self.max_context = int(max_context)
        self.max_batch = int(max_batch)
        self.max_step_tokens = int(max_step_tokens) if max_step_tokens else None
        if self.max_step_tokens is not None and self.max_step_tokens < 1:
            raise ValueError("max_step_tokens must be positive")
        self.eos_token_ids = tuple(eos_token_ids)
        self.bos_token_id = int(bos_token_id)

    # ---- decisions -------------------------------------------------------------------------
    def normalise_prompt(self, prompt: Sequence[int]) -> List[int]:
        ids = [int(t) for t in prompt]
        return ids if ids else [self.bos_token_id]

    def new_token_limit(self, prompt_len: int, max_tokens: int) -> int:
        return max(1, min(int(max_tokens), self.max_context - prompt_len))

    def pages_needed(self, prompt_len: int, max_new: int) -> int:
        # the last drawn token is never fed back, so at most prompt + max_new - 1 positions are cached
        return pages_for(prompt_len + max_new - 1)

    def plan_batches(self, prompts: Sequence[Sequence[int]], params: SamplingParams, free_pages: int) -> List[List[int]]:
        """Request indices grouped into batches, in order: each batch holds at most ``max_batch``
        requests and needs at most ``free_pages`` pages if every request runs to its limit."""
        batches: List[List[int]] = []
        cur: List[int] = []
        used = 0
        for i, p in enumerate(prompts):
            n = len(p)
            if n > self.max_context:
                raise ValueError(f"prompt {i} has {n} tokens, more than the context of {self.max_context}")
            need = self.pages_needed(n, self.new_token_limit(n, params.max_tokens))
            if need > free_pages:
                raise ValueError(
                    f"prompt {i} needs {need} cache pages of {PAGE_TOKENS} tokens but the cache has only {free_pages}")
            if cur and (len(cur) >= self.max_batch or used + need > free_pages):
                batches.append(cur)
                cur, used = [], 0
            cur.append(i)
            used += need
        if cur:
            batches.append(cur)
        return batches

    def plan_prefill(self, lengths: Sequence[int]) -> List[List[Tuple[int, int, int]]]:
        """The steps that bring a batch's prompts in: each a list of (sequence, first token, end) in
        the batch's order, together at most ``max_step_tokens`` tokens.  One step if that fits."""
        budget = self.max_step_tokens
        if budget is None or sum(lengths) <= budget:
            return [[(i, 0, n) for i, n in enumerate(lengths)]]
        steps: List[List[Tuple[int, int, int]]] = [[]]
        used = 0
        for i, n in enumerate(lengths):
            at = 0
            while at < n:
                if used == budget:
                    steps.append([])
                    used = 0
                take = min(n - at, budget - used)
                steps[-1].append((i, at, at + take))
                at += take
                used += take
        return steps

    # ---- the loop ----------------------------------------------------------------------------
    def stream(self, prompts: Sequence[Sequence[int]], params: Optional[SamplingParams] = None) -> Iterator[StreamChunk]:
        params = params or SamplingParams()
        params.validate()
        prompts = [self.normalise_prompt(p) for p in prompts]
        stop_ids = set(self.eos_token_ids) | set(int(t) for t in params.stop_token_ids)
        seed = params.seed if params.seed is not None else int.from_bytes(os.urandom(8), "little")
        for batch in self.plan_batches(prompts, params, self.backend.free_pages()):
            yield from self._run_batch(batch, prompts, params, stop_ids, seed)

    def _run_batch(self, batch: List[int], prompts, params: SamplingParams, stop_ids, seed: int) -> Iterator[StreamChunk]:
        be = self.backend
        live: List[_Live] = []
        launch = getattr(be, "launch_decode", None) if params.repetition_penalty == 1.0 else None
        try:
            for i in batch:
                live.append(_Live(request=i, slot=be.alloc_slot(), prompt=prompts[i],
                                  max_new=self.new_token_limit(len(prompts[i]), params.max_tokens)))
            t0 = time.perf_counter()
            tokens = [0] * len(live)
            for pieces in self.plan_prefill([len(s.prompt) for s in live]):
                # a sequence's first token is drawn in the step that brings the end of its prompt
                ends = [i for i, _, end in pieces if end == len(live[i].prompt)]
                logits = be.step([StepEntry(live[i].slot, live[i].prompt[a:b], (b - a - 1,) if b == len(live[i].prompt) else ())
                                  for i, a, b in pieces])
                if ends:
                    for i, tok in zip(ends, self._draw(logits, [live[i] for i in ends], params, seed)):
                        tokens[i] = tok
            prefill_s = time.perf_counter() - t0
            t_decode = time.perf_counter()

            def take_in(seqs: List[_Live], toks: List[int], free_now: bool):
                """Append each sequence's new token or end the sequence; returns (chunks, still, ended)."""
                chunks, still, ended = [], [], []
                for s, tok in zip(seqs, toks):
                    reason = None
                    if tok in stop_ids:
                        reason = "stop"
                    else:
                        s.generated.append(tok)
                        if len(s.generated) >= s.max_new:
                            reason = "length"
                    if reason is None:
                        still.append(s)
                        chunks.append(StreamChunk(s.request, tok))
                    else:
                        ended.append(s)
                        if free_now:
                            be.free_slot(s.slot)
                            s.slot = -1
                        stats = GenerationResult(
                            token_ids=list(s.generated), prompt_tokens=len(s.prompt),
                            completion_tokens=len(s.generated), finish_reason=reason, prefill_time_s=prefill_s,
                            decode_time_s=time.perf_counter() - t_decode)
                        chunks.append(StreamChunk(s.request, tok, reason, stats))
                return chunks, still, ended

            def give_back(seqs: List[_Live]) -> None:
                for s in seqs:
                    if s.slot >= 0:
                        be.free_slot(s.slot)
                        s.slot = -1

            chunks, live, _ = take_in(live, tokens, True)
            yield from chunks
            pending = None      # a launched decode step for `live` whose tokens have not been read yet
            while live:
                if launch is None:
                    logits = be.step([StepEntry(s.slot, (s.generated[-1],), (0,)) for s in live])
                    tokens = self._draw(logits, live, params, seed)
                    chunks, live, _ = take_in(live, tokens, True)
                    yield from chunks
                    continue
                if pending is None:
                    pending = launch([s.slot for s in live], [s.generated[-1] for s in live], params, seed,
                                     [s.request for s in live], [len(s.generated) for s in live])
                # One step ahead: if no sequence can end by length with the pending token, the step after it is
                # launched now, fed on the device with the tokens the pending step draws.  Only a stop token
                # can then make that work partly useless (the rows of sequences that have just ended).
                ahead = None
                if all(len(s.generated) + 1 < s.max_new for s in live):
                    ahead = launch([s.slot for s in live], None, params, seed, [s.request for s in live],
                                   [len(s.generated) + 1 for s in live])
                tokens = pending.result()
                pending = None
                if ahead is None:
                    chunks, live, _ = take_in(live, tokens, True)
                    yield from chunks
                    continue
                # the slots of sequences that end now stay taken until the step that is in flight is through
                chunks, still, ended = take_in(live, tokens, False)
                yield from chunks
                if not ended:
                    pending = ahead
                    continue
                tokens_ahead = ahead.result()
                give_back(ended)
                keep = {id(s) for s in still}
                pairs = [(s, t) for s, t in zip(live, tokens_ahead) if id(s) in keep]
                chunks, live, _ = take_in([s for s, _ in pairs], [t for _, t in pairs], True)
                yield from chunks
        finally:
            for s in live:
                if s.slot >= 0:
                    be.free_slot(s.slot)
                    s.slot = -1

    def _draw(self, logits, live: List[_Live], params: SamplingParams, seed: int) -> List[int]:
        recent = None
        if params.repetition_penalty != 1.0:
            recent = [s.prompt + s.generated for s in live]
        return self.backend.sample(logits, params, seed, [s.request for s in live], [len(s.generated) for s in live], recent)

    def generate(self, prompts: Sequence[Sequence[int]], params: Optional[SamplingParams] = None) -> List[GenerationResult]:
        results: List[Optional[GenerationResult]] = [None] * len(prompts)
        for chunk in self.stream(prompts, params):
            if chunk.stats is not None:
                results[chunk.request] = chunk.stats
        return results  # type: ignore[return-value]
