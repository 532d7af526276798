#!/usr/bin/env python3
"""A plain PyTorch model of the Qwen3 dense decoder, timed on the same GPU as the engine: the baseline that
``bench.py`` divides by for ``vs_baseline``.

It uses library calls only (``F.linear`` in bfloat16, ``F.scaled_dot_product_attention``, eager mode, a
contiguous cache per batch) and none of this repository's kernels or classes.  The formulas are the
reference's (pygguf_engine/model.py:462-496 attention with q/k-norm before RoPE, 232-251 split-half RoPE,
839-846 SwiGLU, 1025-1042 pre-norm block, 2303-2304 wanted rows before the final norm); the residual stream,
norms and rotation are float32 as there.  Random N(0, 0.02) weights are made on the device; every layer has
matrices of its own, so that a decode step has to read them all from memory as a real model's step does.
"""
from __future__ import annotations

import math
import statistics

import torch
import torch.nn.functional as F
from torch.nn.attention import SDPBackend, sdpa_kernel

# The fused attention kernels that take any key length without preparing a plan per length: with the cuDNN
# backend in the list, a decode loop (one more key every step) spent tens of milliseconds per step on plans.
_SDPA_BACKENDS = [SDPBackend.FLASH_ATTENTION, SDPBackend.EFFICIENT_ATTENTION, SDPBackend.MATH]


class PlainTorchModel:
    def __init__(self, cfg: dict, layers: int, device, dtype=torch.bfloat16, seed: int = 0, share_layers: bool = False):
        g = torch.Generator(device=device).manual_seed(seed)
        self.cfg, self.layers, self.device, self.dtype = cfg, layers, torch.device(device), dtype
        self.h, self.nh, self.nkv, self.d = (cfg["hidden_size"], cfg["num_attention_heads"],
                                             cfg["num_key_value_heads"], cfg["head_dim"])
        self.inter, self.vocab = cfg["intermediate_size"], cfg["vocab_size"]
        self.eps = float(cfg["rms_norm_eps"])

        def mat(r, c):
            return (torch.randn((r, c), generator=g, device=device, dtype=torch.float32) * 0.02).to(dtype)

        def nrm(n):
            return 1.0 + 0.02 * torch.randn((n,), generator=g, device=device, dtype=torch.float32)

        def layer():
            return {"qkv": mat((self.nh + 2 * self.nkv) * self.d, self.h), "o": mat(self.h, self.nh * self.d),
                    "gu": mat(2 * self.inter, self.h), "down": mat(self.h, self.inter), "n1": nrm(self.h),
                    "n2": nrm(self.h), "qn": nrm(self.d), "kn": nrm(self.d)}

        # every layer has weights of its own (a decode step must read them all from memory) unless told otherwise
        one = layer() if share_layers else None
        self.blocks = [one if share_layers else layer() for _ in range(layers)]
        self.embed = mat(self.vocab, self.h)
        self.head = self.embed if cfg.get("tie_word_embeddings", False) else mat(self.vocab, self.h)
        self.final = nrm(self.h)
        half = self.d // 2
        inv = 1.0 / (float(cfg["rope_theta"]) ** (torch.arange(0, self.d, 2, dtype=torch.float32) / self.d))
        self.inv_freq = inv.to(device)
        self.half = half
        self.k_cache = self.v_cache = None

    def alloc_cache(self, batch: int, max_len: int) -> None:
        shape = (self.layers, batch, self.nkv, max_len, self.d)
        self.k_cache = torch.zeros(shape, dtype=self.dtype, device=self.device)
        self.v_cache = torch.zeros(shape, dtype=self.dtype, device=self.device)

    def free_cache(self) -> None:
        self.k_cache = self.v_cache = None

    def _norm(self, x, w):
        x = x.float()
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps) * w

    def _rope(self, x, cos, sin):
        x = x.float()
        x1, x2 = x[..., :self.half], x[..., self.half:]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)

    @torch.inference_mode()
    def forward(self, ids: torch.Tensor, past: int, last_only: bool = True) -> torch.Tensor:
        """``ids`` [B, S] -> float32 logits [B, (1 or S), V]; every sequence holds ``past`` cached tokens."""
        with sdpa_kernel(_SDPA_BACKENDS):
            return self._forward(ids, past, last_only)

    def _forward(self, ids: torch.Tensor, past: int, last_only: bool) -> torch.Tensor:
        B, S = ids.shape
        x = self.embed[ids].float()
        pos = torch.arange(past, past + S, device=self.device, dtype=torch.float32)
        ang = torch.outer(pos, self.inv_freq)
        cos, sin = ang.cos()[None, None], ang.sin()[None, None]
        for li, w in enumerate(self.blocks):
            n = self._norm(x, w["n1"]).to(self.dtype)
            qkv = F.linear(n, w["qkv"])
            q, k, v = qkv.split([self.nh * self.d, self.nkv * self.d, self.nkv * self.d], dim=-1)
            q = q.view(B, S, self.nh, self.d).transpose(1, 2)
            k = k.view(B, S, self.nkv, self.d).transpose(1, 2)
            v = v.view(B, S, self.nkv, self.d).transpose(1, 2)
            q = self._rope(self._norm(q, w["qn"]), cos, sin).to(self.dtype)
            k = self._rope(self._norm(k, w["kn"]), cos, sin).to(self.dtype)
            self.k_cache[li, :B, :, past:past + S] = k
            self.v_cache[li, :B, :, past:past + S] = v
            kk = self.k_cache[li, :B, :, :past + S]
            vv = self.v_cache[li, :B, :, :past + S]
            if S == 1:
                a = F.scaled_dot_product_attention(q, kk, vv, is_causal=False, enable_gqa=True)
            elif past == 0:
                a = F.scaled_dot_product_attention(q, kk, vv, is_causal=True, enable_gqa=True)
            else:
                mask = torch.ones((S, past + S), dtype=torch.bool, device=self.device).tril(past)
                a = F.scaled_dot_product_attention(q, kk, vv, attn_mask=mask, enable_gqa=True)
            a = a.transpose(1, 2).reshape(B, S, self.nh * self.d)
            x = x + F.linear(a, w["o"]).float()
            n = self._norm(x, w["n2"]).to(self.dtype)
            gu = F.linear(n, w["gu"])
            act = F.silu(gu[..., :self.inter].float()) * gu[..., self.inter:].float()
            x = x + F.linear(act.to(self.dtype), w["down"]).float()
        if last_only:
            x = x[:, -1:, :]
        n = self._norm(x, self.final).to(self.dtype)
        return F.linear(n, self.head).float()


def _time(fn, repeats: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(repeats):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    return statistics.median(times)


def measure(cfg: dict, layers: int, *, context: int, batches=(1, 8, 64), prefill_tokens: int = 2048, steps: int = 8,
            warmup: int = 3, device="cuda:0") -> dict:
    """Decode tokens/s (greedy: step + argmax) at each batch with the cache at ``context``, and prefill tokens/s."""
    model = PlainTorchModel(cfg, layers, device)
    out = {}
    gen = torch.Generator(device=device).manual_seed(1)
    for b in batches:
        model.alloc_cache(b, context)
        model.k_cache.normal_(0.0, 0.5)
        model.v_cache.normal_(0.0, 0.5)
        state = {"past": context - steps - warmup - 1,
                 "tok": torch.randint(0, model.vocab, (b, 1), generator=gen, device=device)}

        def step():
            logits = model.forward(state["tok"], state["past"])
            state["tok"] = logits[:, -1].argmax(-1, keepdim=True)
            state["past"] += 1

        for _ in range(warmup):
            step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        out[f"decode_b{b}"] = {"tokens_per_s": round(b * 1000.0 / ms, 2), "ms_per_step": round(ms, 3)}
        model.free_cache()
    if prefill_tokens:
        model.alloc_cache(1, prefill_tokens)
        ids = torch.randint(0, model.vocab, (1, prefill_tokens), generator=gen, device=device)
        ms = _time(lambda: model.forward(ids, 0), repeats=5, warmup=2)
        out["prefill"] = {"tokens_per_s": round(prefill_tokens * 1000.0 / ms, 1), "ms": round(ms, 3),
                          "tokens": prefill_tokens}
        model.free_cache()
    del model
    torch.cuda.empty_cache()
    return out
