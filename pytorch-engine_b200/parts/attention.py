"""Grouped-query softmax attention over the paged cache, with optional per-head q/k RMSNorm,
optional rotary position encoding and an optional sliding window.

Order of operations (pygguf_engine/model.py:462-496): fused q|k|v projection, head split,
q/k-norm over head_dim (before RoPE, not on v), RoPE at position = cached length + row, append of
k, v to the cache, attention with scale ``1/sqrt(head_dim)`` unless the plan gives another
(pygguf_engine/model.py:281-284), merge heads, output projection.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..kernels import ops
from .linear import fuse_rows
from .registry import register
from .spec import CacheRequest, WeightDecl

# keys per partial result in decode: a property of the sequence, never of the batch (measured on the
# tensor-core kernels: 128 / 256 / 512 keys give 4,438 / 5,757 / 6,298 tokens/s at batch 64)
SPLIT_KEYS = 512


@register("mixer", "attention")
class GQAttention:
    """params: ``hidden``, ``n_heads``, ``n_kv_heads``, ``head_dim``, ``qk_norm`` (bool), ``eps``,
    ``scale`` (None: 1/sqrt(head_dim)), ``window`` (None: all keys), ``position`` (name of a position
    encoding of the plan, or None).  weights: ``q_proj, k_proj, v_proj, o_proj`` and, with qk_norm,
    ``q_norm, k_norm``."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    @classmethod
    def weight_decls(cls, params) -> Dict[str, WeightDecl]:
        h, nh, nkv, d = (int(params[k]) for k in ("hidden", "n_heads", "n_kv_heads", "head_dim"))
        decls = {
            "q_proj": WeightDecl((nh * d, h)),
            "k_proj": WeightDecl((nkv * d, h)),
            "v_proj": WeightDecl((nkv * d, h)),
            "o_proj": WeightDecl((h, nh * d)),
        }
        if params.get("qk_norm", False):
            decls["q_norm"] = WeightDecl((d,), "norm")
            decls["k_norm"] = WeightDecl((d,), "norm")
        return decls

    @classmethod
    def cache_request(cls, params) -> Optional[CacheRequest]:
        return CacheRequest(kind="kv", kv_heads=int(params["n_kv_heads"]), head_dim=int(params["head_dim"]),
                            window=params.get("window"))

    def __init__(self, params, weights, runtime, positions=None) -> None:
        self.runtime = runtime
        self.hidden = int(params["hidden"])
        self.n_heads = int(params["n_heads"])
        self.n_kv_heads = int(params["n_kv_heads"])
        self.head_dim = int(params["head_dim"])
        if self.n_heads % self.n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        if self.head_dim > 512:
            raise ValueError(f"head_dim {self.head_dim} is beyond what the attention kernels take (<= 512)")
        self.eps = float(params.get("eps", 1e-6))
        scale = params.get("scale")
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.window = int(params["window"]) if params.get("window") else 0
        self.qkv = fuse_rows(runtime, [weights["q_proj"], weights["k_proj"], weights["v_proj"]])
        self.o_proj = runtime.adopt(weights["o_proj"])
        self.q_norm = self.k_norm = None
        if params.get("qk_norm", False):
            self.q_norm = runtime.adopt(weights["q_norm"], torch.float32)
            self.k_norm = runtime.adopt(weights["k_norm"], torch.float32)
        self.position = None
        self.fused_position = False
        name = params.get("position")
        if name is not None:
            self.position = (positions or {})[name]
            # a rotary encoding with tables is fused into the q/k-norm + append kernel; any other one is
            # applied by its own ``apply(q, k, positions)`` between that kernel's norm and its append
            self.fused_position = bool(getattr(self.position, "fusable_rotary", False))
            if not self.fused_position and not hasattr(self.position, "apply"):
                raise ValueError(f"position encoding {name!r} offers neither tables() nor apply(q, k, positions)")
        self.qkv_dim = (self.n_heads + 2 * self.n_kv_heads) * self.head_dim
        # tensor-core kernels where they take the shape (bfloat16, head size 64 or 128, group <= 16);
        # the generic float32-arithmetic kernels otherwise
        self.use_mma = runtime.is_cuda and ops.attention_mma_supported(runtime.dtype, self.head_dim, self.n_heads,
                                                                       self.n_kv_heads)
        # prefill on tcgen05 where that kernel takes the shape (bfloat16, head size 128, groups up to 32)
        self.use_umma_prefill = runtime.is_cuda and ops.attention_umma_supported(runtime.dtype, self.head_dim,
                                                                                  self.n_heads, self.n_kv_heads)

    def forward(self, x: torch.Tensor, ctx, view, writes_cache: bool = True) -> torch.Tensor:
        rt = self.runtime
        n = x.shape[0]
        qkv = ctx.buffer("attn.qkv", (n, self.qkv_dim), rt.dtype)
        where = (ctx.token_seq, ctx.token_pos, ctx.seq_slot, ctx.seq_qstart, view.page_table, view.num_pages,
                 view.k_pages, view.v_pages)
        if self.fuses_rope_into_product(x, rt):
            # many rows: q/k-norm, rotation and the cache append ride in the epilogue of the q|k|v product (its
            # 256-column tiles are two whole heads), so q|k|v is never written and read again in between
            cos = sin = None
            rotary_dim = 0
            if self.position is not None:
                cos, sin, rotary_dim = self.position.tables()
            ops.gemm_umma2_qkv_rope(x, self.qkv, qkv, self.n_heads, self.n_kv_heads, self.head_dim, self.q_norm, self.k_norm,
                                    self.eps, cos, sin, rotary_dim, *where, writes_cache, rt.status)
        else:
            rt.linear(x, self.qkv, out=qkv)
            self.norm_rotate_append(qkv, n, ctx, view, writes_cache)
        out = ctx.buffer("attn.out", (n, self.n_heads * self.head_dim), rt.dtype)
        self.attend(qkv, out, ctx, view)
        delta = ctx.buffer("attn.delta", (n, self.hidden), rt.dtype)
        rt.linear(out, self.o_proj, out=delta)
        return delta

    def fuses_rope_into_product(self, x: torch.Tensor, rt) -> bool:
        """Whether this step's q|k|v product takes norm, rotation and append into its epilogue: the many-row tcgen05
        pair kernel must be the one that runs (as ``Runtime.linear`` would decide), the position encoding one that
        it can apply (rotary tables over the whole head, or none), the head size 128."""
        if rt.gemm_backend is not None or not rt.fuse_qkv_rope or not rt.pair_gemm or not rt.takes_large_gemm(x, self.qkv):
            return False
        if self.position is not None and not self.fused_position:
            return False
        rotary_dim = self.position.tables()[2] if self.position is not None else 0
        return ops.gemm_umma2_qkv_rope_supported(x, self.qkv, self.n_heads, self.n_kv_heads, self.head_dim, rotary_dim)

    def norm_rotate_append(self, qkv: torch.Tensor, n: int, ctx, view, writes_cache: bool) -> None:
        """q/k-norm, position encoding and cache append on the projected rows, as kernels of their own."""
        rt = self.runtime
        where = (ctx.token_seq, ctx.token_pos, ctx.seq_slot, ctx.seq_qstart, view.page_table, view.num_pages,
                 view.k_pages, view.v_pages)
        shape = (qkv, n, self.n_heads, self.n_kv_heads, self.head_dim)
        if self.position is None or self.fused_position:
            cos = sin = None
            rotary_dim = 0
            if self.position is not None:
                cos, sin, rotary_dim = self.position.tables()
            ops.qk_norm_rope_append(*shape, self.q_norm, self.k_norm, self.eps, cos, sin, rotary_dim, *where,
                                    writes_cache, rt.status)
        else:
            # in the order of the fused kernel: q/k-norm in place, then the position encoding's own code on
            # q and k (views of the fused buffer, [N, heads, head_dim]), then the append of k and v
            if self.q_norm is not None:
                ops.qk_norm_rope_append(*shape, self.q_norm, self.k_norm, self.eps, None, None, 0, *where, False, rt.status)
            qd, kd = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
            self.position.apply(qkv[:, :qd].view(n, self.n_heads, self.head_dim),
                                qkv[:, qd:qd + kd].view(n, self.n_kv_heads, self.head_dim), ctx.token_pos)
            if writes_cache:
                ops.qk_norm_rope_append(*shape, None, None, self.eps, None, None, 0, *where, True, rt.status)

    def attend(self, q: torch.Tensor, out: torch.Tensor, ctx, view) -> None:
        """Attention of the step's queries (the first ``n_heads*head_dim`` features of each row of
        ``q``) over the cache of their sequences."""
        if self.use_umma_prefill and not ctx.decode:
            ops.attention_umma_prefill(
                q, out, ctx.n_seqs, ctx.max_q, self.n_heads, self.n_kv_heads, self.head_dim, self.scale, self.window,
                ctx.seq_qstart, ctx.seq_past, ctx.seq_slot, view.page_table, view.num_pages, view.k_pages, view.v_pages,
                self.runtime.status)
            return
        scratch = None
        max_splits = 0
        split_keys = SPLIT_KEYS
        extra = {}
        if ctx.decode:
            if self.use_mma:
                split_keys, max_splits, floor = ops.attention_mma_decode_ranges(
                    q.device, self.head_dim, ctx.n_seqs, self.n_kv_heads, ctx.max_kv_len, SPLIT_KEYS)
                extra["min_range_keys"] = floor
            else:
                max_splits = ctx.max_splits(split_keys)
            scratch = ctx.buffer(
                "attn.scratch",
                (ops.attention_generic_scratch_floats(ctx.n_seqs, self.n_heads, self.head_dim, max_splits),),
                torch.float32)
        kernel = ops.attention_mma if self.use_mma else ops.attention_generic
        kernel(
            ctx.decode, q, out, ctx.n_seqs, ctx.max_q, self.n_heads, self.n_kv_heads, self.head_dim, self.scale,
            self.window, ctx.seq_qstart, ctx.seq_past, ctx.seq_slot, view.page_table, view.num_pages, view.k_pages,
            view.v_pages, scratch, split_keys, max_splits, self.runtime.status, **extra)
