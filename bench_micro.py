"""Timings of single kernels at the sizes of a configuration, printed as text (``bench.py --micro NAME``).
It sits beside ``bench.py``, outside the package: the package holds what generation runs.

Each case is timed with CUDA events on the launching stream after warm-up.  Cases that compare
kernels call them in turn inside one loop, so that all see the same clocks, and flush L2 between
calls by reading a 256 MB buffer (the matrix products, the decode attention; reading, because a
written buffer leaves 126 MB of dirty lines whose write-back then competes with the timed kernel's
reads: that cost a 201 MB weight stream 20 us) or time a run of calls in a row (the sampler, whose
logits come out of the preceding kernel and sit in L2).
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Sequence

import torch

import importlib

ops = importlib.import_module("pytorch-engine_b200.kernels.ops")


def _flush_buffer(device) -> torch.Tensor:
    return torch.zeros(64 << 20, dtype=torch.int32, device=device)   # 256 MB


def _flush(buffer: torch.Tensor) -> None:
    """Fill L2 with clean lines of ``buffer``."""
    buffer.sum()


def time_in_turn(fns: Sequence[Callable[[], None]], flush: torch.Tensor, rounds: int = 15) -> List[float]:
    """Median microseconds of each callable, called in turn ``rounds`` times with L2 flushed before each call."""
    for f in fns:
        for _ in range(2):
            f()
    times: List[List[float]] = [[] for _ in fns]
    for _ in range(rounds):
        for i, f in enumerate(fns):
            _flush(flush)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            f()
            b.record()
            torch.cuda.synchronize()
            times[i].append(a.elapsed_time(b) * 1e3)
    return [sorted(t)[len(t) // 2] for t in times]


def time_in_a_row(f: Callable[[], None], calls: int = 20) -> float:
    """Microseconds per call over ``calls`` calls in a row."""
    for _ in range(3):
        f()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(calls):
        f()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / calls * 1e3


def gemm(cfg, device, rows: Sequence[int] = (2048, 4096, 1024)) -> None:
    """The tcgen05 products (one SM per tile, a pair of SMs per tile) and the library product."""
    status = torch.zeros(4, dtype=torch.int32, device=device)
    flush = _flush_buffer(device)
    h, i = cfg.hidden_size, cfg.intermediate_size
    qkv = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
    shapes = [("q|k|v", qkv, h, 0), ("o", h, cfg.num_attention_heads * cfg.head_dim, 0), ("gate|up fused", i, h, 1),
              ("down", h, i, 0)]
    for m in rows:
        for name, n, k, pair in shapes:
            x = torch.randn(m, k, device=device).to(torch.bfloat16)
            w = torch.randn(2 * n if pair else n, k, device=device).to(torch.bfloat16)
            out = torch.empty(m, n, device=device, dtype=torch.bfloat16)
            flops = 2.0 * m * (2 * n if pair else n) * k
            fns = [lambda: ops.gemm_umma(x, w, out, status, pair_offset=n if pair else 0),
                   lambda: ops.gemm_umma2(x, w, out, status, pair_offset=n if pair else 0)]
            if not pair:
                fns.append(lambda: torch.mm(x, w.T))
            t = time_in_turn(fns, flush)
            line = (f"M={m} {name} N={n} K={k}: one SM per tile {t[0]:.0f} us ({flops / t[0] / 1e6:.0f} TFLOP/s)  "
                    f"pair of SMs {t[1]:.0f} us ({flops / t[1] / 1e6:.0f} TFLOP/s)")
            if len(t) > 2:
                line += f"  library {t[2]:.0f} us ({flops / t[2] / 1e6:.0f} TFLOP/s)"
            print(line, flush=True)
    print("status word", status.tolist(), flush=True)


def time_in_a_graph(fns: Sequence[Callable[[int], None]], copies: int, rounds: int = 5) -> List[float]:
    """Microseconds per call of each callable ``f(i)`` (``i``: which copy of the operands to use), as one CUDA
    graph of ``copies`` calls each: no host time between the kernels, and with copies that together exceed
    L2 every call streams its operands from memory.  Median of ``rounds`` replays."""
    out = []
    for f in fns:
        for i in range(copies):
            f(i)
        torch.cuda.synchronize()
        stream = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.graph(graph, stream=stream):
            for i in range(copies):
                f(i)
        graph.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(rounds):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3 / copies)
        out.append(sorted(times)[len(times) // 2])
    return out


def gemm_mid(cfg, device, rows: Sequence[int] = (16, 32, 64, 128)) -> None:
    """Products of 9..128 rows, which the engine gives to the library: the library product and this package's
    many-row kernel, each as a CUDA graph of calls that rotate over copies of W larger than L2 together (a single
    call of 15 us cannot be timed from the host: preparing a launch takes as long)."""
    status = torch.zeros(4, dtype=torch.int32, device=device)
    h, i = cfg.hidden_size, cfg.intermediate_size
    qkv = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
    shapes = [("q|k|v", qkv, h), ("o", h, cfg.num_attention_heads * cfg.head_dim), ("down", h, i), ("lm_head", cfg.vocab_size, h)]
    for name, n, k in shapes:
        copies = max(2, min(12, -(-(320 << 20) // (n * k * 2))))
        ws = [torch.randn(n, k, device=device).to(torch.bfloat16) for _ in range(copies)]
        for m in rows:
            x = torch.randn(m, k, device=device).to(torch.bfloat16)
            out = torch.empty(m, n, device=device, dtype=torch.bfloat16)
            t = time_in_a_graph([lambda c: torch.mm(x, ws[c].T, out=out), lambda c: ops.gemm_umma(x, ws[c], out, status)], copies)
            mb = n * k * 2 / 1e6
            print(f"M={m} {name} N={n} K={k} ({mb:.0f} MB x {copies} copies): library {t[0]:.1f} us ({mb / t[0]:.2f} TB/s)  "
                  f"many-row kernel {t[1]:.1f} us", flush=True)
        del ws
    print("status word", status.tolist(), flush=True)


def prefill_attention(cfg, device, lengths: Sequence[int] = (2048, 4096, 8192, 512)) -> None:
    """One prompt through the tcgen05 prefill attention and through the mma.sync one."""
    nh, nkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    for t in lengths:
        pages = (t + 63) // 64 + 2
        kp = (torch.randn(pages, nkv, 64, d, device=device) * 0.5).to(torch.bfloat16)
        vp = (torch.randn(pages, nkv, 64, d, device=device) * 0.5).to(torch.bfloat16)
        table = torch.arange(pages, dtype=torch.int32, device=device).view(1, -1)
        q = torch.randn(t, (nh + 2 * nkv) * d, device=device).to(torch.bfloat16)
        out1 = torch.zeros(t, nh * d, device=device, dtype=torch.bfloat16)
        out2 = torch.zeros_like(out1)
        qstart = torch.tensor([0, t], dtype=torch.int32, device=device)
        past = torch.zeros(1, dtype=torch.int32, device=device)
        slot = torch.zeros(1, dtype=torch.int32, device=device)
        status = torch.zeros(4, dtype=torch.int32, device=device)
        sc = 1 / math.sqrt(d)
        flops = 2.0 * nh * d * t * t     # causal: half of 4 * heads * d * t^2
        line = f"{t} tokens, {nh} x {nkv} heads, d={d}:"
        if ops.attention_umma_supported(torch.bfloat16, d, nh, nkv):
            us = time_in_a_row(lambda: ops.attention_umma_prefill(q, out1, 1, t, nh, nkv, d, sc, 0, qstart, past, slot, table,
                                                                  pages, kp, vp, status), calls=10)
            line += f"  tcgen05 {us:.1f} us ({flops / us / 1e6:.0f} TFLOP/s)"
        if ops.attention_mma_supported(torch.bfloat16, d, nh, nkv):
            us = time_in_a_row(lambda: ops.attention_mma(False, q, out2, 1, t, nh, nkv, d, sc, 0, qstart, past, slot, table,
                                                         pages, kp, vp, None, 0, 0, status), calls=10)
            line += f"  mma.sync {us:.1f} us ({flops / us / 1e6:.0f} TFLOP/s)"
            line += f"  max difference {float((out1.float() - out2.float()).abs().max()):.2e}"
        print(line + f"  status {status.tolist()[0]}", flush=True)


def decode_attention(cfg, device, cases: Sequence[Sequence[int]] = ((8, 4090), (1, 4090), (16, 4090), (64, 4090))) -> None:
    """Split + merge decode attention with ranges of 512 keys, the ranges the engine picks (for a cache of
    this context and of ten times this context), and other even splits."""
    nh, nkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    flush = _flush_buffer(device)
    for batch, length in cases:
        per = (length + 63) // 64 + 1
        pages = batch * per
        kp = (torch.randn(pages, nkv, 64, d, device=device) * 0.5).to(torch.bfloat16)
        vp = (torch.randn(pages, nkv, 64, d, device=device) * 0.5).to(torch.bfloat16)
        table = torch.arange(pages, dtype=torch.int32, device=device).view(batch, per)
        q = torch.randn(batch, (nh + 2 * nkv) * d, device=device).to(torch.bfloat16)
        qstart = torch.arange(batch + 1, dtype=torch.int32, device=device)
        past = torch.full((batch,), length - 1, dtype=torch.int32, device=device)
        slot = torch.arange(batch, dtype=torch.int32, device=device)
        status = torch.zeros(4, dtype=torch.int32, device=device)
        max_kv = -(-length // 64) * 64

        def make(split_keys, max_splits, least=0):
            out = torch.zeros(batch, nh * d, device=device, dtype=torch.bfloat16)
            scratch = torch.zeros(ops.attention_generic_scratch_floats(batch, nh, d, max_splits), device=device)
            return lambda: ops.attention_mma(True, q, out, batch, 1, nh, nkv, d, 1 / math.sqrt(d), 0, qstart, past, slot,
                                             table, pages, kp, vp, scratch, split_keys, max_splits, status,
                                             min_range_keys=least)

        picked = ops.attention_mma_decode_ranges(torch.device(device), d, batch, nkv, max_kv, 512)
        # the engine's pick for a cache that allows sequences ten times as long: the least range size keeps
        # this context's ranges as they are, its spare blocks return at once
        roomy = ops.attention_mma_decode_ranges(torch.device(device), d, batch, nkv, 10 * max_kv, 512)
        configs = [(512, -(-max_kv // 512)), picked, roomy] + [(0, n) for n in (2, 4, 8, 16) if batch * nkv * n <= 1200]
        t = time_in_turn([make(*c) for c in configs], flush, rounds=12)
        nbytes = 2 * batch * length * nkv * d * 2
        cells = [f"{c}: {us:.1f} us ({nbytes / us / 1e6:.2f} TB/s)" for c, us in zip(configs, t)]
        print(f"batch {batch} context {length} (split_keys, ranges[, least keys]): " + "  ".join(cells) +
              f"  [engine picks {picked}; {roomy} in a cache for {10 * max_kv} keys]",
              flush=True)


def sampler(cfg, device, batches: Sequence[int] = (1, 8, 64)) -> None:
    """The sampler with and without the scratch that lets it cut rows into chunks."""
    v = cfg.vocab_size
    settings = [("greedy", 0.0, 0, 1.0, 0.0), ("temperature 0.7, top-k 40, top-p 0.95, min-p 0.05", 0.7, 40, 0.95, 0.05),
                ("temperature only", 0.7, 0, 1.0, 0.0), ("top-p 0.95 only", 0.7, 0, 0.95, 0.0)]
    for b in batches:
        logits = torch.randn(b, v, device=device) * 3
        req = torch.arange(b, dtype=torch.int32, device=device)
        step = torch.zeros(b, dtype=torch.int32, device=device)
        out = torch.empty(b, dtype=torch.int32, device=device)
        for name, t, k, p, m in settings:
            need = ops.sample_scratch_bytes(b, v, t, k, p, m)
            scratch = torch.empty(need, dtype=torch.uint8, device=device) if need else None
            one = time_in_a_row(lambda: ops.sample(logits, t, k, p, m, 1, req, step, out))
            two = time_in_a_row(lambda: ops.sample(logits, t, k, p, m, 1, req, step, out, scratch=scratch)) if need else None
            print(f"batch {b} vocabulary {v} {name}: one kernel {one:.1f} us" +
                  (f", two kernels {two:.1f} us" if two is not None else ", no two-kernel path"), flush=True)


def rope_append(cfg, device, cases: Sequence[Sequence[int]] = ((2048, 1), (2048, 4), (512, 1), (8192, 2), (8, 8))) -> None:
    """q/k-norm + rotation + append of a step of N tokens in B sequences (calls in a row: the rows it reads were
    just written by the q|k|v product and sit in L2, as here)."""
    nh, nkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    for n, b in cases:
        ld = (nh + 2 * nkv) * d
        qkv = torch.randn(n, ld, device=device).to(torch.bfloat16)
        qw, kw = torch.ones(d, device=device), torch.ones(d, device=device)
        cos, sin = torch.randn(8192, d // 2, device=device), torch.randn(8192, d // 2, device=device)
        per = n // b
        token_seq = torch.arange(n, device=device, dtype=torch.int32) // per
        past = 4000 if per == 1 else 0
        token_pos = (torch.arange(n, device=device, dtype=torch.int32) % per) + past
        seq_slot = torch.arange(b, device=device, dtype=torch.int32)
        qstart = torch.arange(b + 1, device=device, dtype=torch.int32) * per
        pages_per = 8192 // 64
        table = torch.arange(b * pages_per, device=device, dtype=torch.int32).view(b, pages_per)
        kp = torch.zeros(b * pages_per, nkv, 64, d, device=device, dtype=torch.bfloat16)
        vp = torch.zeros_like(kp)
        status = torch.zeros(4, dtype=torch.int32, device=device)
        us = time_in_a_row(lambda: ops.qk_norm_rope_append(qkv, n, nh, nkv, d, qw, kw, 1e-6, cos, sin, d, token_seq, token_pos,
                                                           seq_slot, qstart, table, b * pages_per, kp, vp, True, status), calls=20)
        moved = n * ld * 2 + n * (nh + nkv) * d * 2 + n * 2 * nkv * d * 2     # rows read, q and k written back, k and v to the cache
        print(f"{n} tokens in {b} sequence(s), {nh} x {nkv} heads, d={d}: {us:.1f} us ({moved / us / 1e6:.2f} TB/s)  "
              f"status {status.tolist()[0]}", flush=True)


CASES: Dict[str, Callable] = {"rope_append": rope_append, "gemm_mid": gemm_mid, "gemm": gemm, "prefill_attention": prefill_attention, "decode_attention": decode_attention, "sampler": sampler}
