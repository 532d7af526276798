"""The step function: a batch of sequences that started together, from the cache, to logits.

``ModelRunner.step(entries)`` runs exactly the tokens it is given, as one batch: for each entry the
tokens follow what that entry's slot already holds.  Prompts of unequal lengths go in one step;
later steps bring one token per live sequence.  Logits come back only for the wanted positions.
Nothing is padded in the eager path; the CUDA-graph path for one-token steps replays a graph
captured for exactly that number of sequences, with slots and lengths read from device memory
(the reference feeds its decode graphs the position the same way, pygguf_engine/model.py:197-209,
1743-1872).  Generation, the Python entry point and trace replay all go through this one function.
"""
from __future__ import annotations

import gc
from typing import Dict, List, Optional, Sequence

import torch

from ..cache import PagedCache
from ..kernels import ops
from .batch import BufferPool, PinnedStager, StepContext, StepEntry
from .model import DecoderModel


class _DecodeGraph:
    def __init__(self, graph, ctx: StepContext, logits: torch.Tensor, pool: BufferPool, launches: int) -> None:
        self.graph = graph
        self.ctx = ctx
        self.logits = logits
        self.pool = pool
        self.launches = launches  # kernels of this package recorded in the graph


class ModelRunner:
    def __init__(self, model: DecoderModel, cache: PagedCache, *, cuda_graphs: bool = True) -> None:
        self.model = model
        self.cache = cache
        self.runtime = model.runtime
        self.pool = BufferPool(self.runtime.device)
        self.stager = PinnedStager(self.runtime.device)
        self.cuda_graphs = bool(cuda_graphs) and self.runtime.is_cuda and model.graph_safe()
        self._graphs: Dict[int, _DecodeGraph] = {}
        self.steps_run = 0
        self.kernel_launch_estimate = 0

    # ---- slots -------------------------------------------------------------------------
    def alloc_slot(self) -> int:
        return self.cache.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self.cache.free_slot(slot)

    # ---- the step ------------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry], check: bool = True) -> torch.Tensor:
        """Logits (float32, ``[wanted positions in entry order, vocab]``) after feeding each entry's
        tokens.  The returned tensor may be overwritten by the next step."""
        entries = list(entries)
        if not entries:
            raise ValueError("a step needs at least one sequence")
        seen = set()
        pasts: List[int] = []
        for e in entries:
            if e.slot in seen:
                raise ValueError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if len(e.tokens) == 0:
                raise ValueError(f"slot {e.slot} brings no token in this step")
            pasts.append(self.cache.length(e.slot))
        ints, n_tokens, n_want = StepContext.pack_meta(entries, pasts)   # raises on a wanted place outside the step
        # make room before anything runs: on a failure the pages taken so far go back and the cache is as it was
        self._reserve_all([(e.slot, past + len(e.tokens)) for e, past in zip(entries, pasts)])
        n_seqs = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        decode = all(q == 1 for q in q_lens)
        if decode and self.cuda_graphs and n_want == n_seqs and all(tuple(e.want) == (0,) for e in entries):
            logits = self._step_graph(ints, n_seqs)
        else:
            ctx = StepContext(self.runtime, self.pool, n_tokens=n_tokens, n_seqs=n_seqs, max_q=max(q_lens),
                              decode=decode, n_want=n_want,
                              # decode: the longest sequence the cache allows, as in the captured graphs, so that how a
                              # sequence's keys are cut into ranges never depends on the other sequences' lengths
                              max_kv_len=self.cache.max_seq_len if decode else max(p + q for p, q in zip(pasts, q_lens)))
            self.stager.send(ints, ctx.meta)
            ops.batch_expand(ctx.seq_qstart, ctx.seq_past, n_seqs, ctx.token_seq, ctx.token_pos)
            logits = self.model.forward(ctx, self.cache)
        for e, past in zip(entries, pasts):
            self.cache.commit(e.slot, past + len(e.tokens))
        self.steps_run += 1
        if check:
            self.runtime.raise_on_status()
        return logits

    def can_step_from_device_tokens(self, n_seqs: int) -> bool:
        return self.cuda_graphs and n_seqs in self._graphs

    def step_from_device_tokens(self, slots: Sequence[int], device_tokens: torch.Tensor) -> torch.Tensor:
        """One decode step for ``slots`` whose input tokens are ``device_tokens`` (int32, on the device, one
        per slot): the graph captured for this many sequences is replayed with its token buffer filled by
        a device-to-device copy, so the host never sees the tokens on the way in."""
        n = len(slots)
        g = self._graphs[n]
        pasts = [self.cache.length(s) for s in slots]
        self._reserve_all([(s, past + 1) for s, past in zip(slots, pasts)])
        g.ctx.tokens.copy_(device_tokens[:n], non_blocking=True)
        self.stager.send(list(slots) + pasts + list(range(n + 1)) + list(range(n)), g.ctx.meta[n:])
        g.graph.replay()
        ops.count_replay(g.launches)
        for s, past in zip(slots, pasts):
            self.cache.commit(s, past + 1)
        self.steps_run += 1
        return g.logits

    def _reserve_all(self, wanted) -> None:
        """Reserve pages for every (slot, new length); all or nothing."""
        done = []
        try:
            for slot, length in wanted:
                self.cache.reserve(slot, length)
                done.append(slot)
        except Exception:
            for slot in done:
                self.cache.release_reserved(slot)
            raise

    def _step_graph(self, meta_ints, n_seqs: int) -> torch.Tensor:
        g = self._graphs.get(n_seqs)
        if g is None:
            g = self._capture(torch.tensor(meta_ints, dtype=torch.int32), n_seqs)
        else:
            self.stager.send(meta_ints, g.ctx.meta)
            g.graph.replay()
            ops.count_replay(g.launches)
        return g.logits

    def _capture(self, host_meta: torch.Tensor, n_seqs: int) -> _DecodeGraph:
        """Capture one decode step for exactly ``n_seqs`` sequences.  The step runs exactly once, eagerly
        (which also warms up library handles and kernel attributes): recording it into the graph afterwards
        executes nothing, and the eager run's logits are handed over to the graph's output buffer.  So a mixer
        that folds each token into a state of fixed size sees this step's tokens once, as in every other step."""
        pool = BufferPool(self.runtime.device)
        ctx = StepContext(self.runtime, pool, n_tokens=n_seqs, n_seqs=n_seqs, max_q=1, decode=True,
                          max_kv_len=self.cache.max_seq_len, n_want=n_seqs)
        ctx.meta.copy_(host_meta)
        stream = torch.cuda.Stream(device=self.runtime.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            ops.batch_expand(ctx.seq_qstart, ctx.seq_past, n_seqs, ctx.token_seq, ctx.token_pos)
            eager_logits = self.model.forward(ctx, self.cache)  # the step itself
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize(self.runtime.device)
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        # No collector run in mid-capture: one that frees what an engine dropped earlier left behind (pinned
        # buffers, events) makes CUDA calls that a capturing stream forbids, and the capture is lost.
        gc.collect()
        collecting = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
                ops.batch_expand(ctx.seq_qstart, ctx.seq_past, n_seqs, ctx.token_seq, ctx.token_pos)
                logits = self.model.forward(ctx, self.cache)
        finally:
            if collecting:
                gc.enable()
        launches = ops.launch_count() - before
        if logits.data_ptr() != eager_logits.data_ptr():
            logits.copy_(eager_logits)
        g = _DecodeGraph(graph, ctx, logits, pool, launches)
        self._graphs[n_seqs] = g
        return g

    def workspace_bytes(self) -> int:
        return self.pool.nbytes() + sum(g.pool.nbytes() for g in self._graphs.values())
