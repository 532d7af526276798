"""What parts share at run time: device, run dtype, the status word, and the matrix product.

``Runtime.linear`` is the one place where ``y = x W^T`` is computed.  The reference computes its
unquantised linears with a library call (``F.linear``, pygguf_engine/quant_kernels.py:1836); here
the library product (cuBLAS through ``torch.mm``) stands wherever the package's own tensor-core
kernels do not take the shape, and the float32 mode always runs in true float32 (TF32 is switched
off around the call).
"""
from __future__ import annotations

import os
from typing import Dict, Optional, Tuple

import torch

from ..kernels import KernelError, ops

STATUS_MESSAGES = {
    1: "a token id is outside the embedding table (token row {0}, id {1}, vocabulary {2})",
    2: "a cache page number is outside the pool ({0}, page {1}, {2})",
    3: "a position is beyond the position tables or the page table (token {0}, position {1}, limit {2})",
    4: "a bounded wait inside a kernel ran out (where {0}, detail {1}, {2})",
    5: "a slot number is outside the cache ({0}, {1}, {2})",
}


class PendingTokens:
    """Tokens (and the status word) on their way to the host; ``result()`` waits and returns the tokens,
    raising if a kernel reported an error."""

    def __init__(self, runtime: "Runtime") -> None:
        self.runtime = runtime
        self.host = torch.empty(4 + runtime.max_result_rows, dtype=torch.int32, pin_memory=runtime.is_cuda)
        self.event = torch.cuda.Event() if runtime.is_cuda else None
        self.n = 0

    def start(self, n: int) -> None:
        self.n = n
        self.host[:4 + n].copy_(self.runtime._status_and_tokens[:4 + n], non_blocking=True)
        if self.event is not None:
            self.event.record()

    def result(self):
        if self.event is not None:
            self.event.synchronize()
        vals = self.host[:4 + self.n].tolist()
        if vals[0] != 0:
            self.runtime.status.zero_()
            msg = STATUS_MESSAGES.get(vals[0], "kernel status {0}").format(*vals[1:4])
            raise KernelError(f"a kernel reported an error during the step: {msg}")
        return vals[4:]


def large_gemm_fill(rows: int, cols: int, sms: int) -> float:
    """Share of busy tile slots when ``rows x cols`` outputs are cut into 256 x 256 tiles and run in
    waves of one tile per pair of SMs: 96 tiles on 74 pairs need two waves and fill 0.65 of them."""
    tiles = -(-rows // 256) * -(-cols // 256)
    pairs = max(1, sms // 2)
    waves = -(-tiles // pairs)
    return tiles / (waves * pairs)


class Runtime:
    def __init__(self, device, dtype: torch.dtype) -> None:
        self.device = torch.device(device)
        if dtype not in (torch.float32, torch.bfloat16):
            raise KernelError(f"run dtype must be float32 or bfloat16, got {dtype}")
        self.dtype = dtype
        self.is_cuda = self.device.type == "cuda"
        # the status word (4 ints) and, right behind it, room for the tokens a sampler draws: one
        # device-to-host copy then brings both
        self.max_result_rows = 8192
        self._status_and_tokens = torch.zeros(4 + self.max_result_rows, dtype=torch.int32, device=self.device)
        self.status = self._status_and_tokens[:4]
        self.token_area = self._status_and_tokens[4:]
        self._host_result = None
        self._pending_ring = None
        self._pending_next = 0
        self._adopted: Dict[Tuple[int, torch.dtype], torch.Tensor] = {}
        self.gemm_backend = None  # a callable (x, weight, out, out_dtype) -> tensor or None that takes over products
        self.own_small_gemm = True  # products with few rows run on csrc/gemm_smallm.cu
        self.small_gemm_rows = 8    # up to this many rows (measured: beyond it the library product is faster)
        # products with many rows run on csrc/gemm_umma.cu (tcgen05 + TMA); in between, and for shapes it
        # refuses, the library product stands (measured: with fewer rows too few tiles exist to fill the SMs)
        self.own_large_gemm = True
        self.large_gemm_rows = 1024
        self.large_gemm_min_fill = 0.8   # least share of the waves of tiles that does work (see takes_large_gemm)
        self.pair_gemm = True       # large products on tcgen05 cta_group::2
        # q/k-norm, rotation and cache append in the epilogue of the q|k|v product where the pair kernel runs it
        # (PE_B200_FUSE_QKV_ROPE=0 keeps them kernels of their own, for comparisons)
        self.fuse_qkv_rope = os.environ.get("PE_B200_FUSE_QKV_ROPE", "1") != "0"

    # ---- weights -------------------------------------------------------------------------
    def adopt(self, tensor: torch.Tensor, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """The tensor on the run device in ``dtype`` (default: the run dtype), converted once even if
        several parts use it (tied embedding and output head share one copy)."""
        dtype = dtype or self.dtype
        key = (id(tensor), dtype)
        got = self._adopted.get(key)
        if got is None:
            got = tensor.to(device=self.device, dtype=dtype).contiguous()
            self._adopted[key] = got
        return got

    def forget_adopted(self) -> None:
        self._adopted.clear()

    # ---- status word -----------------------------------------------------------------------
    def raise_on_status(self) -> None:
        """Read the kernels' status word (one small device-to-host copy) and raise if it is set."""
        s = self.status.tolist()
        if s[0] != 0:
            self.status.zero_()
            msg = STATUS_MESSAGES.get(s[0], "kernel status {0}").format(*s[1:])
            raise KernelError(f"a kernel reported an error during the step: {msg}")

    def takes_small_gemm(self, x: torch.Tensor, weight: torch.Tensor) -> bool:
        return (self.own_small_gemm and x.dim() == 2 and x.shape[0] <= self.small_gemm_rows
                and ops.gemm_smallm_supported(x, weight))

    def takes_large_gemm(self, x: torch.Tensor, weight: torch.Tensor, pair_offset: int = 0) -> bool:
        rows = 9 if pair_offset else self.large_gemm_rows   # the fused gate wins at every size above the small kernel's
        if not (self.own_large_gemm and x.dim() == 2 and x.shape[0] >= rows
                and ops.gemm_umma_supported(x, weight, pair_offset)):
            return False
        # A plain product whose 256 x 256 tiles leave the last wave of SM pairs mostly idle goes to the
        # library, which has smaller tiles to choose from (8B shape, 1,536 rows, down projection: 96 tiles
        # on 74 pairs took 133 us against 103 us).
        return bool(pair_offset) or large_gemm_fill(x.shape[0], weight.shape[0], ops.sm_count(x.device)) >= self.large_gemm_min_fill

    def fetch_tokens(self, n: int):
        """The first ``n`` ints of ``token_area`` as a list, after checking the status word: one
        device-to-host copy for both (the copy waits for the step's kernels)."""
        if self._host_result is None:
            self._host_result = torch.empty(4 + self.max_result_rows, dtype=torch.int32,
                                            pin_memory=self.is_cuda)
        host = self._host_result[:4 + n]
        host.copy_(self._status_and_tokens[:4 + n], non_blocking=True)
        if self.is_cuda:
            torch.cuda.current_stream(self.device).synchronize()
        vals = host.tolist()
        if vals[0] != 0:
            self.status.zero_()
            msg = STATUS_MESSAGES.get(vals[0], "kernel status {0}").format(*vals[1:4])
            raise KernelError(f"a kernel reported an error during the step: {msg}")
        return vals[4:]

    def fetch_tokens_async(self, n: int) -> "PendingTokens":
        """Start the copy of the status word and the first ``n`` ints of ``token_area`` to the host and
        return at once; ``result()`` of the returned handle waits for it.  The device may go on and
        overwrite ``token_area`` meanwhile: the copy is ordered before whatever is launched next."""
        if self._pending_ring is None:
            self._pending_ring = [PendingTokens(self) for _ in range(4)]
            self._pending_next = 0
        h = self._pending_ring[self._pending_next]
        self._pending_next = (self._pending_next + 1) % len(self._pending_ring)
        h.start(n)
        return h

    # ---- matrix product ----------------------------------------------------------------------
    def linear(self, x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None,
               out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """``x [M, K] @ weight [N, K]^T -> [M, N]``."""
        if not self.is_cuda:
            raise KernelError("this package computes on a CUDA device only; there is no CPU path")
        if self.gemm_backend is not None:
            y = self.gemm_backend(x, weight, out, out_dtype)
            if y is not None:
                return y
        if self.takes_large_gemm(x, weight):
            if out is None:
                out = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype or x.dtype, device=x.device)
            # two SMs per 256 x 256 tile (csrc/gemm_umma2.cu): measured 3-6 % faster than one SM per
            # 128 x 256 tile on the plain products; the fused gate|up product stays on gemm_umma.cu
            pair = self.pair_gemm and ops.gemm_umma2_supported(x, weight)
            (ops.gemm_umma2 if pair else ops.gemm_umma)(x, weight, out, self.status)
            return out
        if self.takes_small_gemm(x, weight):
            # a handful of rows: the package's weight-streaming kernel (csrc/gemm_smallm.cu)
            if out is None:
                out = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype or x.dtype, device=x.device)
            ops.gemm_smallm(x, weight, out)
            return out
        if x.dtype == torch.float32:
            prev = torch.backends.cuda.matmul.allow_tf32
            if prev:
                torch.backends.cuda.matmul.allow_tf32 = False
            try:
                return torch.mm(x, weight.t(), out=out) if out is not None else torch.mm(x, weight.t())
            finally:
                if prev:
                    torch.backends.cuda.matmul.allow_tf32 = True
        # library product in bfloat16: keep its reductions in float32
        prev = torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction
        if prev:
            torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        try:
            if out_dtype is not None and out_dtype != x.dtype:
                y = torch.mm(x, weight.t(), out_dtype=out_dtype)
                if out is not None:
                    out.copy_(y)
                    return out
                return y
            return torch.mm(x, weight.t(), out=out) if out is not None else torch.mm(x, weight.t())
        finally:
            if prev:
                torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = True
