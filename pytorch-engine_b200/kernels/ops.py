"""Tensor-level wrappers of the CUDA entry points.  Every op requires CUDA tensors."""
from __future__ import annotations

from typing import Optional

import torch

from .lib import PE_BF16, PE_F32, KernelError, check, library


def dtype_tag(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return PE_F32
    if dtype == torch.bfloat16:
        return PE_BF16
    raise KernelError(f"unsupported dtype {dtype}: the kernels run in float32 or bfloat16")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("the kernels of this package run on CUDA tensors only; got a CPU tensor")
    return t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle (the raw query is several times cheaper than building a
    ``torch.cuda.Stream`` object, and this runs once per launch)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


# How many kernels of this library were launched (a replayed CUDA graph counts its captured kernels
# through ``count_replay``); benchmarks report it.
_LAUNCHES = 0


def _count(n: int = 1) -> None:
    global _LAUNCHES
    _LAUNCHES += n


def launch_count() -> int:
    return _LAUNCHES


def count_replay(n: int) -> None:
    _count(n)


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> None:
    _need(ids.dtype == torch.int32 and out.dtype == torch.float32, "embed_gather: ids int32, out float32")
    _need(table.is_contiguous() and out.is_contiguous() and ids.is_contiguous(), "embed_gather: contiguous tensors")
    n, hidden = out.shape
    check(library().pe_embed_gather(dtype_tag(table.dtype), _ptr(table), _ptr(ids), _ptr(out), n, hidden,
                                    table.shape[0], _ptr(status), _stream()), "embed_gather")
    _count(1)


def rmsnorm_residual(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, out: torch.Tensor,
                     eps: float, rows: Optional[torch.Tensor] = None) -> None:
    """``out = rmsnorm(residual (+ delta)) * weight``; see csrc/rmsnorm.cu for the two modes."""
    _need(residual.dtype == torch.float32 and weight.dtype == torch.float32, "rmsnorm: stream and weight float32")
    _need(residual.is_contiguous() and out.is_contiguous(), "rmsnorm: contiguous tensors")
    if delta is not None:
        _need(delta.dtype == out.dtype and delta.is_contiguous() and delta.shape == residual.shape,
              "rmsnorm: delta must match the stream's shape and the output dtype")
    dim = residual.shape[-1]
    n_rows = out.shape[0]
    if rows is not None:
        _need(rows.dtype == torch.int32 and rows.numel() == n_rows, "rmsnorm: rows int32, one per output row")
    else:
        _need(n_rows == residual.shape[0], "rmsnorm: output rows must match the stream")
    check(library().pe_rmsnorm_residual(dtype_tag(out.dtype), _ptr(residual), _ptr(delta), _ptr(weight), _ptr(out),
                                        _ptr(rows), n_rows, dim, float(eps), _stream()), "rmsnorm_residual")
    _count(1)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float) -> None:
    _need(x.is_contiguous() and out.is_contiguous() and weight.dtype == torch.float32, "rmsnorm: contiguous, weight f32")
    dim = x.shape[-1]
    check(library().pe_rmsnorm(dtype_tag(x.dtype), _ptr(x), _ptr(weight), _ptr(out), x.numel() // dim, dim, float(eps),
                               _stream()), "rmsnorm")
    _count(1)


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    _need(gate_up.is_contiguous() and out.is_contiguous(), "silu_mul: contiguous tensors")
    n, two_i = gate_up.shape
    _need(two_i == 2 * out.shape[1] and out.shape[0] == n and out.dtype == gate_up.dtype, "silu_mul: shapes")
    check(library().pe_silu_mul(dtype_tag(gate_up.dtype), _ptr(gate_up), _ptr(out), n, out.shape[1], _stream()), "silu_mul")
    _count(1)


def batch_expand(seq_qstart: torch.Tensor, seq_past: torch.Tensor, n_seqs: int, token_seq: torch.Tensor,
                 token_pos: torch.Tensor) -> None:
    check(library().pe_batch_expand(_ptr(seq_qstart), _ptr(seq_past), n_seqs, _ptr(token_seq), _ptr(token_pos),
                                    _stream()), "batch_expand")
    _count(1)


def qk_norm_rope_append(qkv: torch.Tensor, n_tokens: int, n_heads: int, n_kv_heads: int, head_dim: int,
                        q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], eps: float,
                        cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int,
                        token_seq: torch.Tensor, token_pos: torch.Tensor, seq_slot: torch.Tensor,
                        seq_qstart: torch.Tensor, page_table: Optional[torch.Tensor], num_pages: int, k_pages: Optional[torch.Tensor],
                        v_pages: Optional[torch.Tensor], write_cache: bool, status: torch.Tensor) -> None:
    _need(qkv.stride(-1) == 1, "qk_norm_rope_append: rows of qkv must be contiguous")
    table_rows = 0 if cos is None else cos.shape[0]
    check(library().pe_qk_norm_rope_append(
        dtype_tag(qkv.dtype), _ptr(qkv), qkv.stride(0), n_tokens, n_heads, n_kv_heads, head_dim,
        _ptr(q_norm_w), _ptr(k_norm_w), float(eps), _ptr(cos), _ptr(sin), rotary_dim if cos is not None else 0,
        table_rows, _ptr(token_seq), _ptr(token_pos), _ptr(seq_slot), _ptr(seq_qstart), _ptr(page_table),
        0 if page_table is None else page_table.shape[1], num_pages, _ptr(k_pages), _ptr(v_pages),
        1 if write_cache else 0, _ptr(status), _stream()), "qk_norm_rope_append")
    _count(1)


def attention_generic_scratch_floats(n_seqs: int, n_heads: int, head_dim: int, max_splits: int) -> int:
    return int(library().pe_attention_generic_scratch_floats(n_seqs, n_heads, head_dim, max_splits))


def attention_generic(decode: bool, q: torch.Tensor, out: torch.Tensor, n_seqs: int, max_q: int, n_heads: int,
                      n_kv_heads: int, head_dim: int, scale: float, window: int, seq_qstart: torch.Tensor,
                      seq_past: torch.Tensor, seq_slot: torch.Tensor, page_table: torch.Tensor, num_pages: int,
                      k_pages: torch.Tensor, v_pages: torch.Tensor, scratch: Optional[torch.Tensor], split_keys: int,
                      max_splits: int, status: torch.Tensor) -> None:
    _need(q.stride(-1) == 1 and out.stride(-1) == 1, "attention: rows must be contiguous")
    _need(q.dtype == out.dtype == k_pages.dtype, "attention: q, out and the cache must share a dtype")
    check(library().pe_attention_generic(
        dtype_tag(q.dtype), 1 if decode else 0, _ptr(q), q.stride(0), _ptr(out), out.stride(0), n_seqs, max_q,
        n_heads, n_kv_heads, head_dim, float(scale), int(window), _ptr(seq_qstart), _ptr(seq_past), _ptr(seq_slot),
        _ptr(page_table), page_table.shape[1], num_pages, _ptr(k_pages), _ptr(v_pages), _ptr(scratch), split_keys,
        max_splits, _ptr(status), _stream()), "attention_generic")
    _count(2 if decode else 1)


def attention_mma_supported(dtype: torch.dtype, head_dim: int, n_heads: int, n_kv_heads: int) -> bool:
    """Whether the tensor-core attention kernels (csrc/attention_mma.cu) take this shape."""
    return dtype == torch.bfloat16 and bool(library().pe_attention_mma_supported(head_dim, n_heads, n_kv_heads))


def attention_mma(decode: bool, q: torch.Tensor, out: torch.Tensor, n_seqs: int, max_q: int, n_heads: int,
                  n_kv_heads: int, head_dim: int, scale: float, window: int, seq_qstart: torch.Tensor,
                  seq_past: torch.Tensor, seq_slot: torch.Tensor, page_table: torch.Tensor, num_pages: int,
                  k_pages: torch.Tensor, v_pages: torch.Tensor, scratch: Optional[torch.Tensor], split_keys: int,
                  max_splits: int, status: torch.Tensor, min_range_keys: int = 0) -> None:
    """Same contract as ``attention_generic``, bfloat16 only, head sizes 64 and 128, groups up to 16.
    With ``split_keys`` 0 a sequence's keys are shared out evenly over ``max_splits`` ranges of whole pages,
    each of at least ``min_range_keys`` keys."""
    _need(q.stride(-1) == 1 and out.stride(-1) == 1, "attention: rows must be contiguous")
    _need(q.dtype == out.dtype == k_pages.dtype == torch.bfloat16, "attention_mma: bfloat16 tensors only")
    check(library().pe_attention_mma(
        1 if decode else 0, _ptr(q), q.stride(0), _ptr(out), out.stride(0), n_seqs, max_q, n_heads, n_kv_heads,
        head_dim, float(scale), int(window), _ptr(seq_qstart), _ptr(seq_past), _ptr(seq_slot), _ptr(page_table),
        page_table.shape[1], num_pages, _ptr(k_pages), _ptr(v_pages), _ptr(scratch), split_keys, max_splits,
        int(min_range_keys), _ptr(status), _stream()), "attention_mma")
    _count(2 if decode else 1)


def gemm_smallm_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether csrc/gemm_smallm.cu takes ``x [M, K] @ weight [N, K]^T``: bfloat16, M <= 16, K % 8 == 0."""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[0] <= 16
            and x.shape[1] % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and weight.is_contiguous())


def gemm_smallm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, pair_offset: int = 0) -> None:
    """``out[M, N] = x @ weight^T`` (out bfloat16 or float32).  With ``pair_offset`` = I the weight holds
    gate rows then up rows and ``out[M, I] = silu(x @ gate^T) * (x @ up^T)``."""
    _need(gemm_smallm_supported(x, weight), "gemm_smallm: needs bfloat16, M <= 16, K % 8 == 0, contiguous rows")
    _need(out.stride(-1) == 1 and out.dtype in (torch.bfloat16, torch.float32), "gemm_smallm: out bfloat16 or float32")
    m, k = x.shape
    n = out.shape[1]
    _need(weight.shape[1] == k and weight.shape[0] == (2 * n if pair_offset else n) and out.shape[0] == m,
          "gemm_smallm: shapes do not match")
    _need(pair_offset in (0, n), "gemm_smallm: pair_offset must be 0 or the output width")
    check(library().pe_gemm_smallm(_ptr(x), x.stride(0), _ptr(weight), _ptr(out), out.stride(0), m, n, k,
                                   1 if out.dtype == torch.float32 else 0, pair_offset, sm_count(x.device), _stream()), "gemm_smallm")
    _count(1)


_SM_COUNT = {}


def sm_count(device) -> int:
    idx = torch.device(device).index or 0
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SM_COUNT[idx]


def gemm_umma_supported(x: torch.Tensor, weight: torch.Tensor, pair_offset: int = 0) -> bool:
    """Whether csrc/gemm_umma.cu (tcgen05 + TMA) takes ``x [M, K] @ weight^T``: bfloat16, K % 8 == 0."""
    if not (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and weight.is_contiguous() and x.data_ptr() % 16 == 0):
        return False
    n = weight.shape[0] // 2 if pair_offset else weight.shape[0]
    return bool(library().pe_gemm_umma_supported(x.shape[0], n, x.shape[1], pair_offset))


def gemm_umma(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, status: torch.Tensor, pair_offset: int = 0) -> None:
    """``out[M, N] = x @ weight^T`` on the tcgen05 tensor cores (out bfloat16 or float32); with
    ``pair_offset`` = I: ``out[M, I] = silu(x @ gate^T) * (x @ up^T)`` for weight = [gate; up]."""
    _need(gemm_umma_supported(x, weight, pair_offset), "gemm_umma: needs bfloat16, K % 8 == 0, dense weight rows")
    _need(out.stride(-1) == 1 and out.dtype in (torch.bfloat16, torch.float32), "gemm_umma: out bfloat16 or float32")
    m, k = x.shape
    n = out.shape[1]
    _need(weight.shape[1] == k and weight.shape[0] == (2 * n if pair_offset else n) and out.shape[0] == m,
          "gemm_umma: shapes do not match")
    _need(not pair_offset or out.dtype == torch.bfloat16, "gemm_umma: the fused gate writes bfloat16")
    check(library().pe_gemm_umma(_ptr(x), x.stride(0), _ptr(weight), _ptr(out), out.stride(0), m, n, k,
                                 1 if out.dtype == torch.float32 else 0, pair_offset, sm_count(x.device), _ptr(status),
                                 _stream()), "gemm_umma")
    _count(1)


def gemm_umma2_supported(x: torch.Tensor, weight: torch.Tensor, pair_offset: int = 0) -> bool:
    """Whether csrc/gemm_umma2.cu takes the product: as ``gemm_umma_supported``, and K % 64 == 0."""
    if not gemm_umma_supported(x, weight, pair_offset):
        return False
    n = weight.shape[0] // 2 if pair_offset else weight.shape[0]
    return bool(library().pe_gemm_umma2_supported(x.shape[0], n, x.shape[1], pair_offset))


def gemm_umma2(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, status: torch.Tensor, pair_offset: int = 0) -> None:
    """``gemm_umma`` with two SMs per 256 x 256 output tile (csrc/gemm_umma2.cu, tcgen05 cta_group::2)."""
    _need(gemm_umma2_supported(x, weight, pair_offset), "gemm_umma2: needs bfloat16, K % 64 == 0, dense weight rows")
    _need(out.stride(-1) == 1 and out.dtype in (torch.bfloat16, torch.float32), "gemm_umma2: out bfloat16 or float32")
    m, k = x.shape
    n = out.shape[1]
    _need(weight.shape[1] == k and weight.shape[0] == (2 * n if pair_offset else n) and out.shape[0] == m,
          "gemm_umma2: shapes do not match")
    _need(not pair_offset or out.dtype == torch.bfloat16, "gemm_umma2: the fused gate writes bfloat16")
    check(library().pe_gemm_umma2(_ptr(x), x.stride(0), _ptr(weight), _ptr(out), out.stride(0), m, n, k,
                                  1 if out.dtype == torch.float32 else 0, pair_offset, sm_count(x.device), _ptr(status),
                                  _stream()), "gemm_umma2")
    _count(1)


def gemm_umma2_qkv_rope_supported(x: torch.Tensor, weight: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                                  rotary_dim: int) -> bool:
    """Whether the q|k|v projection of this layer can run with q/k-norm, rotation and cache append in its epilogue
    (csrc/gemm_umma2.cu, mode 3): bfloat16, head size 128, the whole head rotated or none of it, K % 64 == 0."""
    if not gemm_umma2_supported(x, weight):
        return False
    return bool(library().pe_gemm_umma2_qkv_rope_supported(x.shape[0], x.shape[1], n_heads, n_kv_heads, head_dim, rotary_dim))


def gemm_umma2_qkv_rope(x: torch.Tensor, weight: torch.Tensor, qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                        q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], eps: float,
                        cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int, token_seq: torch.Tensor,
                        token_pos: torch.Tensor, seq_slot: torch.Tensor, seq_qstart: torch.Tensor,
                        page_table: Optional[torch.Tensor], num_pages: int, k_pages: Optional[torch.Tensor],
                        v_pages: Optional[torch.Tensor], write_cache: bool, status: torch.Tensor) -> None:
    """``x @ weight^T`` (the fused q|k|v projection) with what ``qk_norm_rope_append`` does in the product's epilogue:
    ``qkv[:, :n_heads * head_dim]`` gets the normalised, rotated queries; keys and values go to the cache only."""
    _need(gemm_umma2_qkv_rope_supported(x, weight, n_heads, n_kv_heads, head_dim, rotary_dim if cos is not None else 0),
          "gemm_umma2_qkv_rope: needs bfloat16, head size 128, whole-head rotation, K % 64 == 0")
    _need(qkv.dtype == torch.bfloat16 and qkv.stride(-1) == 1 and qkv.shape[0] == x.shape[0], "gemm_umma2_qkv_rope: qkv rows")
    _need(weight.shape[0] == (n_heads + 2 * n_kv_heads) * head_dim, "gemm_umma2_qkv_rope: weight rows")
    m, k = x.shape
    check(library().pe_gemm_umma2_qkv_rope(
        _ptr(x), x.stride(0), _ptr(weight), _ptr(qkv), qkv.stride(0), m, k, n_heads, n_kv_heads, head_dim,
        _ptr(q_norm_w), _ptr(k_norm_w), float(eps), _ptr(cos), _ptr(sin), rotary_dim if cos is not None else 0,
        0 if cos is None else cos.shape[0], _ptr(token_seq), _ptr(token_pos), _ptr(seq_slot), _ptr(seq_qstart),
        _ptr(page_table), 0 if page_table is None else page_table.shape[1], num_pages, _ptr(k_pages), _ptr(v_pages),
        1 if write_cache else 0, sm_count(x.device), _ptr(status), _stream()), "gemm_umma2_qkv_rope")
    _count(1)


def decode_ranges(slots: int, pairs: int, max_kv_len: int, split_keys: int) -> tuple:
    """(split_keys, max_splits, min_range_keys) for a decode attention whose SMs hold ``slots`` blocks at a
    time and that has ``pairs`` (sequence, kv head) pairs; split_keys 0 means that each sequence's keys
    are shared out evenly over max_splits ranges (in whole pages, of at least min_range_keys keys).
    When one wave of blocks can hold at least two ranges per pair, that many ranges are used, but not
    more than ranges of ``split_keys`` keys would give (measured: the blocks of a second, partly filled
    wave cost more than longer ranges do, and more, shorter ranges only add merge work).  With more
    pairs than that there are several waves anyway, and ranges of about four times ``split_keys`` keys
    were measured best (batch 64 at 4,096 keys: 169 us with two ranges, 179 us with eight).  The same
    two sizes are the least a range may have: ``max_kv_len`` is the longest sequence the cache allows,
    and a sequence far shorter than that is not to be cut into as many ranges."""
    pairs = max(1, pairs)
    fixed = max(1, -(-max_kv_len // split_keys))
    per_pair = slots // pairs
    if per_pair < 2:
        return 0, max(1, min(fixed, -(-max_kv_len // (4 * split_keys)))), 4 * split_keys
    return 0, min(per_pair, fixed), split_keys


def attention_mma_decode_ranges(device: torch.device, head_dim: int, n_seqs: int, n_kv_heads: int, max_kv_len: int,
                                split_keys: int) -> tuple:
    """``decode_ranges`` for csrc/attention_mma.cu on this device."""
    slots = sm_count(device) * int(library().pe_attention_mma_decode_blocks_per_sm(head_dim))
    return decode_ranges(slots, n_seqs * n_kv_heads, max_kv_len, split_keys)


def attention_umma_supported(dtype: torch.dtype, head_dim: int, n_heads: int, n_kv_heads: int) -> bool:
    """Whether the tcgen05 prefill attention (csrc/attention_umma.cu) takes this shape."""
    return dtype == torch.bfloat16 and bool(library().pe_attention_umma_supported(head_dim, n_heads, n_kv_heads))


_WORK_COUNTERS = {}


def _work_counter(device: torch.device) -> torch.Tensor:
    """Two zero ints per (device, stream) for kernels that hand out work through a counter; the kernels
    leave them zero.  Launches on one stream run one after the other, so they may share a counter."""
    key = (device.index or 0, _stream())
    t = _WORK_COUNTERS.get(key)
    if t is None:
        t = torch.zeros(2, dtype=torch.int32, device=device)
        _WORK_COUNTERS[key] = t
    return t


def attention_umma_prefill(q: torch.Tensor, out: torch.Tensor, n_seqs: int, max_q: int, n_heads: int, n_kv_heads: int,
                           head_dim: int, scale: float, window: int, seq_qstart: torch.Tensor, seq_past: torch.Tensor,
                           seq_slot: torch.Tensor, page_table: torch.Tensor, num_pages: int, k_pages: torch.Tensor,
                           v_pages: torch.Tensor, status: torch.Tensor) -> None:
    """Prefill attention on tcgen05 (bfloat16, head size 128, groups up to 32); ``q`` holds the step's
    query rows (the first ``n_heads * head_dim`` features of each row of the fused q|k|v buffer)."""
    _need(q.stride(-1) == 1 and out.stride(-1) == 1, "attention: rows must be contiguous")
    _need(q.dtype == out.dtype == k_pages.dtype == torch.bfloat16, "attention_umma: bfloat16 tensors only")
    check(library().pe_attention_umma_prefill(
        _ptr(q), q.stride(0), q.shape[0], _ptr(out), out.stride(0), n_seqs, max_q, n_heads, n_kv_heads, head_dim,
        float(scale), int(window), _ptr(seq_qstart), _ptr(seq_past), _ptr(seq_slot), _ptr(page_table),
        page_table.shape[1], num_pages, _ptr(k_pages), _ptr(v_pages), sm_count(q.device), _ptr(_work_counter(q.device)), _ptr(status), _stream()),
        "attention_umma_prefill")
    _count(1)


def sample_scratch_bytes(n_rows: int, vocab: int, temperature: float, top_k: int, top_p: float = 1.0,
                         min_p: float = 0.0) -> int:
    """Bytes of scratch with which ``sample`` runs as two kernels (many blocks per row) for these
    settings: greedy, no filter at all, or a small top-k; 0 if it has no such path for them."""
    return int(library().pe_sample_scratch_bytes(int(n_rows), int(vocab), float(temperature), int(top_k),
                                                 float(top_p), float(min_p)))


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, min_p: float, seed: int,
           row_request: torch.Tensor, row_step: torch.Tensor, out_tokens: torch.Tensor,
           scratch: Optional[torch.Tensor] = None) -> None:
    """One token per row.  ``scratch`` (uint8, at least ``sample_scratch_bytes``) lets greedy and small
    top-k draws cut each row into chunks first; the drawn tokens are the same either way except
    where float32 sums in another order move an entry across a top-p threshold."""
    _need(logits.dtype == torch.float32 and logits.stride(-1) == 1, "sample: float32 logits with contiguous rows")
    n, vocab = logits.shape
    two = scratch is not None and scratch.numel() * scratch.element_size() >= max(1, sample_scratch_bytes(n, vocab, temperature, top_k, top_p, min_p))
    check(library().pe_sample(_ptr(logits), logits.stride(0), n, vocab, float(temperature), int(top_k), float(top_p),
                              float(min_p), int(seed) & ((1 << 64) - 1), _ptr(row_request), _ptr(row_step),
                              _ptr(out_tokens), _ptr(scratch) if two else None,
                              scratch.numel() * scratch.element_size() if two else 0, _stream()), "sample")
    _count(2 if two and sample_scratch_bytes(n, vocab, temperature, top_k, top_p, min_p) > 0 else 1)


def repetition_penalty(logits: torch.Tensor, recent: torch.Tensor, recent_count: torch.Tensor, penalty: float) -> None:
    n, vocab = logits.shape
    check(library().pe_repetition_penalty(_ptr(logits), logits.stride(0), n, vocab, _ptr(recent), recent.shape[1],
                                          _ptr(recent_count), float(penalty), _stream()), "repetition_penalty")
    _count(1)


def wait_poll_seconds(device, polls: int = 20000) -> float:
    """Seconds that one poll of an mbarrier takes when the phase it asks for is not complete (csrc/wait_probe.cu):
    ``polls`` polls of a barrier on which nothing arrives, timed on the device."""
    out = torch.zeros(2, dtype=torch.int64, device=device)
    check(library().pe_wait_probe(_ptr(out), int(polls), _stream()), "wait_probe")
    _count(1)
    ns, passed = out.tolist()
    _need(passed == 0, "wait_probe: a poll of a barrier that nothing arrives on passed")
    return ns * 1e-9 / polls


def wait_limit_seconds(device) -> float:
    """The longest that a bounded wait inside a kernel of this library lasts before it gives up."""
    return int(library().pe_wait_limit_polls()) * wait_poll_seconds(device)
