"""The device sampler: float32 logits rows -> one token id per row (see csrc/sampling.cu)."""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..kernels import ops
from .params import SamplingParams

RECENT_WINDOW = 256  # the reference penalises the unique ids among the last 256 tokens (engine.py:94)


class Sampler:
    def __init__(self, device, runtime=None) -> None:
        """With a ``runtime`` the drawn tokens land behind its status word and come back together with
        it in one copy (``Runtime.fetch_tokens``), which also raises if a kernel reported an error."""
        self.device = torch.device(device)
        self.runtime = runtime
        self._stager = None     # made at the first draw, with the two halves of _meta
        self._meta = None
        self._meta_turn = 0
        self._scratch = None

    def _scratch_for(self, logits: torch.Tensor, params: SamplingParams) -> Optional[torch.Tensor]:
        """Scratch for the sampler's two-kernel path, grown when a larger batch comes."""
        need = ops.sample_scratch_bytes(logits.shape[0], logits.shape[1], params.temperature, params.top_k,
                                        params.top_p, params.min_p)
        if need == 0:
            return None
        if self._scratch is None or self._scratch.numel() < need:
            self._scratch = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=self.device)
        return self._scratch

    def _launch_into_token_area(self, logits, params, seed, requests, steps) -> None:
        from ..engine.batch import PinnedStager
        rt = self.runtime
        n = logits.shape[0]
        if self._stager is None:
            self._stager = PinnedStager(self.device)
            # two halves used in turn: a launched sampler may still read one while the next is being filled
            self._meta = torch.empty(2, 2 * rt.max_result_rows, dtype=torch.int32, device=self.device)
        self._meta_turn ^= 1
        meta = self._meta[self._meta_turn, :2 * n]
        self._stager.send(list(requests) + list(steps), meta)
        ops.sample(logits, params.temperature, params.top_k, params.top_p, params.min_p, seed, meta[:n], meta[n:],
                   rt.token_area[:n], scratch=self._scratch_for(logits, params))

    def sample_async(self, logits: torch.Tensor, params: SamplingParams, seed: int, requests: Sequence[int],
                     steps: Sequence[int]):
        """Launch the draw and the copy of its tokens to the host; returns a handle whose ``result()``
        waits for them.  The tokens also stay in the runtime's token area on the device, where the next
        decode step can take them from without the host in between.  (No repetition penalty here: it
        needs the token history on the host.)"""
        rt = self.runtime
        n = logits.shape[0]
        if rt is None or n > rt.max_result_rows:
            raise ValueError("sample_async needs a runtime and at most %d rows" % (rt.max_result_rows if rt else 0))
        self._launch_into_token_area(logits, params, seed, requests, steps)
        return rt.fetch_tokens_async(n)

    def sample(self, logits: torch.Tensor, params: SamplingParams, seed: int, requests: Sequence[int],
               steps: Sequence[int], recent: Optional[Sequence[Sequence[int]]] = None) -> List[int]:
        """One token per row of ``logits``.  ``requests[r]`` and ``steps[r]`` key row r's random
        numbers (the request's index and how many tokens it has drawn so far); ``recent[r]`` is the
        row's token history for the repetition penalty."""
        n = logits.shape[0]
        if n == 0:
            return []
        if params.repetition_penalty != 1.0 and recent is not None:
            logits = logits.clone()
            rec = torch.zeros((n, RECENT_WINDOW), dtype=torch.int32)
            cnt = torch.zeros((n,), dtype=torch.int32)
            for r, hist in enumerate(recent):
                tail = list(hist)[-RECENT_WINDOW:]
                cnt[r] = len(tail)
                if tail:
                    rec[r, :len(tail)] = torch.tensor(tail, dtype=torch.int32)
            ops.repetition_penalty(logits, rec.to(self.device), cnt.to(self.device), params.repetition_penalty)
        rt = self.runtime
        if rt is not None and n <= rt.max_result_rows:
            self._launch_into_token_area(logits, params, seed, requests, steps)
            return rt.fetch_tokens(n)
        meta = torch.tensor([list(requests), list(steps)], dtype=torch.int32).to(self.device)
        out = torch.empty((n,), dtype=torch.int32, device=self.device)
        ops.sample(logits, params.temperature, params.top_k, params.top_p, params.min_p, seed, meta[0], meta[1], out,
                   scratch=self._scratch_for(logits, params))
        return out.tolist()
