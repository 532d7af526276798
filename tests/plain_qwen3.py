"""Plain, slow restatement of the Qwen3 dense decoder, used only as the tests' oracle.

Whole sequences, float32, no cache, no batching, one function per part.  It shares no code with
the package: it reads ``config.json`` as a plain dict and tensors by their checkpoint names.

Every function cites the place in binief/pytorch-engine (paths within that project) whose formula
it restates.  ``tests/golden/make_golden.py`` compares this file once with that project's own
model code on the CPU and commits the small outputs, so the formulas here are anchored on it.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch


# --------------------------------------------------------------------------------------------
# storage precision
# --------------------------------------------------------------------------------------------
def stored(x: torch.Tensor, store: Optional[torch.dtype]) -> torch.Tensor:
    """``x`` as it reads back after being stored in ``store`` (None: float32, nothing happens).

    All arithmetic in this file is float32.  A run in bfloat16 stores its activations in 16 bits
    between operations, as the reference stores them in float16 (pygguf_engine/model.py:1025 norm
    output, pygguf_engine/quant_kernels.py:1836 linear output, pygguf_engine/model.py:241 rotated q/k,
    pygguf_engine/kv_cache.py:861 attention output, pygguf_engine/quant_kernels.py:1474 gated product);
    ``store=torch.bfloat16`` rounds at those places and nowhere else: the residual stream
    (pygguf_engine/model.py:1033-1042), softmax, norms' statistics and the logits stay float32.
    Norm followed by rotation is one computation here and rounds once, after the rotation.
    """
    return x if store is None else x.to(store).to(torch.float32)


# --------------------------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps) * w`` over the last dim, all in float32.

    pygguf_engine/quant_kernels.py:1548 (``F.rms_norm(x.float(), (D,), w, eps)``), the Triton form
    at pygguf_engine/quant_kernels.py:831-833, weight held in float32 at pygguf_engine/model.py:63.
    """
    x = x.to(torch.float32)
    var = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * weight.to(torch.float32)


def rope_inv_freq(rotary_dim: int, theta: float) -> torch.Tensor:
    """``1 / theta^(2j / rotary_dim)``, j = 0 .. rotary_dim/2 - 1, float32.

    pygguf_engine/model.py:147-156 (the unscaled branch).
    """
    idx = torch.arange(0, rotary_dim, 2, dtype=torch.float32)
    return 1.0 / (float(theta) ** (idx / rotary_dim))


def rope_cos_sin(positions: torch.Tensor, rotary_dim: int, theta: float):
    """cos/sin of ``position * inv_freq`` as float32 ``[S, rotary_dim/2]``.

    pygguf_engine/model.py:183-185 (positions as float32, outer product, then cos and sin).
    """
    freqs = torch.outer(positions.to(torch.float32), rope_inv_freq(rotary_dim, theta))
    return torch.cos(freqs), torch.sin(freqs)


def rope_rotate_neox(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rotary_dim: int) -> torch.Tensor:
    """Split-half (NeoX) rotation of the first ``rotary_dim`` features; the rest pass through.

    ``x`` is ``[S, heads, d]``; ``cos``/``sin`` are ``[S, rotary_dim/2]``.
    pygguf_engine/model.py:232-251 (``neox_style`` branch 237-241, pass-through 249-250).
    """
    x = x.to(torch.float32)
    half = rotary_dim // 2
    x1 = x[..., :half]
    x2 = x[..., half:rotary_dim]
    c = cos[:, None, :]
    s = sin[:, None, :]
    rotated = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)
    if rotary_dim < x.shape[-1]:
        return torch.cat([rotated, x[..., rotary_dim:]], dim=-1)
    return rotated


def causal_gqa_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    scale: float,
    window: Optional[int] = None,
    q_start: int = 0,
) -> torch.Tensor:
    """Softmax attention of ``q [S, nh, d]`` over ``k, v [T, nkv, d]`` with a causal mask.

    Query row ``i`` sits at position ``q_start + i``; key ``j`` at position ``j``.
    * key visible iff ``kpos <= qpos`` (pygguf_engine/kv_cache.py:2192; flash kernel 833);
    * with a window also ``kpos > qpos - window`` (pygguf_engine/kv_cache.py:2189-2190);
    * scores ``q.k * scale``, softmax over visible keys, ``p.v`` (pygguf_engine/kv_cache.py:2280-2305);
    * query head ``h`` reads kv head ``h // group`` (pygguf_engine/kv_cache.py:756, 2265-2270).
    """
    S, nh, d = q.shape
    T, nkv, _ = k.shape
    group = nh // nkv
    q = q.to(torch.float32)
    k = k.to(torch.float32)
    v = v.to(torch.float32)
    qpos = torch.arange(q_start, q_start + S)[:, None]
    kpos = torch.arange(T)[None, :]
    visible = kpos <= qpos
    if window is not None:
        visible = visible & (kpos > qpos - window)
    out = torch.empty(S, nh, d, dtype=torch.float32)
    for h in range(nh):
        kv_h = h // group
        scores = (q[:, h, :] @ k[:, kv_h, :].T) * scale
        scores = scores.masked_fill(~visible, float("-inf"))
        p = torch.softmax(scores, dim=-1)
        out[:, h, :] = p @ v[:, kv_h, :]
    return out


def swiglu(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor,
           store: Optional[torch.dtype] = None) -> torch.Tensor:
    """``(silu(x Wg^T) * (x Wu^T)) Wd^T`` with ``silu(z) = z / (1 + exp(-z))``.

    pygguf_engine/model.py:839-846 and pygguf_engine/quant_kernels.py:1467-1475.  The reference's
    row scale ``max(1, max|inter| / 16384)`` guards a float16 overflow and cancels exactly
    (divide before ``down``, multiply after), so it does not appear in float32.
    """
    x = x.to(torch.float32)
    gate = stored(x @ w_gate.to(torch.float32).T, store)
    up = stored(x @ w_up.to(torch.float32).T, store)
    inter = stored((gate / (1.0 + torch.exp(-gate))) * up, store)
    return stored(inter @ w_down.to(torch.float32).T, store)


def attention_layer(
    x_normed: torch.Tensor,
    w: Dict[str, torch.Tensor],
    prefix: str,
    *,
    n_heads: int,
    n_kv_heads: int,
    head_dim: int,
    eps: float,
    theta: float,
    window: Optional[int],
    store: Optional[torch.dtype] = None,
) -> torch.Tensor:
    """q/k/v projections, per-head q/k RMSNorm, RoPE, causal GQA attention, output projection.

    pygguf_engine/model.py:462-496: projections 462, head split 467-469, q/k-norm before RoPE and
    not on v 471-474, RoPE 476, attention 485-491, merge heads 492, o_proj 496; softmax scale
    ``1/sqrt(head_dim)`` at pygguf_engine/model.py:284.
    """
    S = x_normed.shape[0]
    f = lambda name: w[f"{prefix}.self_attn.{name}.weight"].to(torch.float32)
    q = stored(x_normed @ f("q_proj").T, store).view(S, n_heads, head_dim)
    k = stored(x_normed @ f("k_proj").T, store).view(S, n_kv_heads, head_dim)
    v = stored(x_normed @ f("v_proj").T, store).view(S, n_kv_heads, head_dim)
    q = rms_norm(q, f("q_norm"), eps)
    k = rms_norm(k, f("k_norm"), eps)
    cos, sin = rope_cos_sin(torch.arange(S), head_dim, theta)
    q = stored(rope_rotate_neox(q, cos, sin, head_dim), store)
    k = stored(rope_rotate_neox(k, cos, sin, head_dim), store)
    o = stored(causal_gqa_attention(q, k, v, 1.0 / math.sqrt(head_dim), window=window), store)
    return stored(o.reshape(S, n_heads * head_dim) @ f("o_proj").T, store)


def decoder_block(x: torch.Tensor, w: Dict[str, torch.Tensor], layer: int, cfg: dict, window: Optional[int],
                  store: Optional[torch.dtype] = None) -> torch.Tensor:
    """Pre-norm block: ``h = x + attn(norm(x))``; ``out = h + mlp(norm(h))``; residual in float32.

    pygguf_engine/model.py:1025-1042.
    """
    p = f"model.layers.{layer}"
    eps = float(cfg["rms_norm_eps"])
    n = stored(rms_norm(x, w[f"{p}.input_layernorm.weight"], eps), store)
    a = attention_layer(
        n, w, p,
        n_heads=cfg["num_attention_heads"],
        n_kv_heads=cfg["num_key_value_heads"],
        head_dim=cfg["head_dim"],
        eps=eps,
        theta=float(cfg["rope_theta"]),
        window=window,
        store=store,
    )
    h = x + a
    n2 = stored(rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], eps), store)
    f = swiglu(n2, w[f"{p}.mlp.gate_proj.weight"], w[f"{p}.mlp.up_proj.weight"], w[f"{p}.mlp.down_proj.weight"], store)
    return h + f


def layer_window(cfg: dict, layer: int) -> Optional[int]:
    """The sliding window of a layer, or None: ``layer_types`` if config.json lists them, else
    layers from ``max_window_layers`` on when ``use_sliding_window`` is set.  The reference's dense
    path has no window of its own (its ring cache serves another head, pygguf_engine/kv_cache.py:1614-1620);
    the mask is the one of pygguf_engine/kv_cache.py:2189-2190.
    """
    if not cfg.get("use_sliding_window", False) or not cfg.get("sliding_window"):
        return None
    types = cfg.get("layer_types")
    if types is not None:
        return int(cfg["sliding_window"]) if types[layer] == "sliding_attention" else None
    return int(cfg["sliding_window"]) if layer >= int(cfg.get("max_window_layers", 0)) else None


def forward_logits(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int],
                   store: Optional[torch.dtype] = None) -> torch.Tensor:
    """Logits ``[S, V]`` (float32) at every position of one whole sequence.  ``store``: see ``stored``.

    pygguf_engine/model.py:2235-2305: embedding to float32 2237, blocks 2276-2292, final norm 2189-2192,
    output head 2206-2211 (the embedding table when tied, pygguf_engine/model.py:1678-1683), float32 2214.
    """
    cfg = dict(cfg)
    cfg.setdefault("num_key_value_heads", cfg["num_attention_heads"])
    cfg.setdefault("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    x = w["model.embed_tokens.weight"].to(torch.float32)[ids]
    for layer in range(cfg["num_hidden_layers"]):
        x = decoder_block(x, w, layer, cfg, layer_window(cfg, layer), store)
    n = stored(rms_norm(x, w["model.norm.weight"], float(cfg["rms_norm_eps"])), store)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return n @ head.to(torch.float32).T


def load_folder(folder: str):
    """(config dict, {name: tensor}) of a model folder, read with the safetensors library only."""
    from safetensors import safe_open

    with open(os.path.join(folder, "config.json")) as fh:
        cfg = json.load(fh)
    tensors: Dict[str, torch.Tensor] = {}
    index = os.path.join(folder, "model.safetensors.index.json")
    files = ["model.safetensors"]
    if os.path.isfile(index):                       # a folder written in shards
        with open(index) as fh:
            files = sorted(set(json.load(fh)["weight_map"].values()))
    for fname in files:
        with safe_open(os.path.join(folder, fname), framework="pt", device="cpu") as fh:
            for name in fh.keys():
                tensors[name] = fh.get_tensor(name)
    return cfg, tensors


# --------------------------------------------------------------------------------------------
# generation and sampling, restated
# --------------------------------------------------------------------------------------------
_M64 = (1 << 64) - 1


def _mix64(z: int) -> int:
    """splitmix64 finaliser on a Python int (the engine's counter-based generator, restated)."""
    z = (z + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def uniform_for(seed: int, request: int, step: int, index: int) -> float:
    """The uniform number in (0, 1) that the engine draws for vocabulary entry ``index``."""
    key = _mix64((seed & _M64) ^ _mix64(((request & 0xFFFFFFFF) << 32) | (step & 0xFFFFFFFF)))
    bits = _mix64((key + index) & _M64) >> 40  # 24 bits
    return (bits + 0.5) / float(1 << 24)


def filter_logits(
    logits: torch.Tensor,
    *,
    temperature: float,
    top_k: int = 0,
    top_p: float = 1.0,
    min_p: float = 0.0,
    repetition_penalty: float = 1.0,
    recent_tokens: Sequence[int] = (),
):
    """The reference's filter chain on one row; returns (penalised logits, probabilities or None).

    pygguf_engine/engine.py:91-134: repetition penalty on the unique ids of the last 256 tokens
    (negative logits times p, others divided by p) 92-97; greedy below 1e-5 99-100; divide by the
    temperature 102; top-k 104-108; softmax 110; min-p against the largest probability 112-114;
    top-p drops entries whose preceding mass exceeds it 116-124; renormalise 126-133.
    """
    logits = logits.to(torch.float32).clone()
    if repetition_penalty != 1.0 and len(recent_tokens) > 0:
        for t in set(list(recent_tokens)[-256:]):
            logits[t] = logits[t] * repetition_penalty if logits[t] < 0 else logits[t] / repetition_penalty
    if temperature <= 1e-5:
        return logits, None
    scaled = logits * (1.0 / temperature)
    keep = torch.ones_like(scaled, dtype=torch.bool)
    if 0 < top_k < scaled.numel():
        kth = torch.topk(scaled, top_k).values[-1]
        keep &= scaled >= kth
    probs = torch.softmax(scaled.masked_fill(~keep, float("-inf")), dim=-1)
    if min_p > 0.0:
        probs = torch.where(probs < min_p * probs.max(), torch.zeros_like(probs), probs)
    if 0.0 < top_p < 1.0:
        sp, si = torch.sort(probs, descending=True, stable=True)
        cum = torch.cumsum(sp, dim=-1)
        sp = sp.masked_fill((cum - sp) > top_p, 0.0)
        probs = torch.zeros_like(probs).scatter_(0, si, sp)
    total = probs.sum()
    if total > 0:
        probs = probs / total
    else:
        probs = torch.zeros_like(probs)
        probs[int(torch.argmax(logits))] = 1.0
    return logits, probs


def gumbel_scores(logits: torch.Tensor, *, seed: int, request: int, step: int, **filters) -> Optional[torch.Tensor]:
    """``log p_i - log(-log u_i)`` for every kept entry (minus infinity for the dropped ones) with the engine's
    counter-based uniform numbers, float64; None for a greedy draw."""
    _, probs = filter_logits(logits, **filters)
    if probs is None:
        return None
    logp = torch.log(probs.to(torch.float64))
    scores = torch.full_like(logp, -float("inf"))
    for i in range(probs.numel()):
        if probs[i] <= 0:
            continue
        u = uniform_for(seed, request, step, i)
        scores[i] = float(logp[i]) - math.log(-math.log(u))
    return scores


def sample_token(logits: torch.Tensor, *, seed: int, request: int, step: int, **filters) -> int:
    """Greedy argmax, or a draw from the filtered distribution by the Gumbel-max rule with the
    engine's counter-based uniform numbers: ``argmax(log p_i - log(-log u_i))`` over kept entries.
    (The reference draws with ``torch.multinomial``, pygguf_engine/engine.py:149; its stream depends
    on the batch layout, so the engine keys its numbers by request and step instead.)
    """
    scores = gumbel_scores(logits, seed=seed, request=request, step=step, **filters)
    if scores is None:
        pen, _ = filter_logits(logits, **filters)
        return int(torch.argmax(pen))
    return int(torch.argmax(scores))         # the first of equal scores, as a loop with ">" would keep


def check_drawn_tokens(cfg: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], tokens: Sequence[int], *,
                       seed: int, request: int, margin: float, **filters) -> int:
    """Follows ``tokens`` (what an engine drew for ``prompt``) and checks each against this file's own draw
    from this file's own logits, with the same seed, request number and step.  A token may differ only where
    the two best scores lie within ``margin`` of each other (the engine's logits differ from these by rounding,
    so a near tie may fall the other way; its choice must then be the runner-up) .  Returns how many differed."""
    toks = list(prompt)
    differed = 0
    for j, tok in enumerate(tokens):
        row = forward_logits(cfg, w, toks)[-1]
        if filters.get("repetition_penalty", 1.0) != 1.0:
            filters["recent_tokens"] = list(toks)    # the penalty looks at the prompt and what has been drawn so far
        scores = gumbel_scores(row, seed=seed, request=request, step=j, **filters)
        if scores is None:
            scores = filter_logits(row, **filters)[0].to(torch.float64)
        best = torch.topk(scores, 2)
        if int(best.indices[0]) != tok:
            assert float(best.values[0] - best.values[1]) < margin and int(best.indices[1]) == tok, (
                f"request {request}, token {j}: the engine drew {tok}, the plain draw is {int(best.indices[0])} "
                f"(score {float(best.values[0]):.6f}, runner-up {int(best.indices[1])} at {float(best.values[1]):.6f})")
            differed += 1
        toks.append(tok)
    return differed


def generate_greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], max_tokens: int,
                    stop_ids: Sequence[int] = ()) -> List[int]:
    """Greedy continuation by re-running the whole sequence for every new token.

    pygguf_engine/engine.py:637-651 (first token from the last prompt row; a stop token ends the
    sequence and is not part of the output) and 695, 860-867, 891-893 (length limit).
    """
    toks = list(prompt)
    out: List[int] = []
    while len(out) < max_tokens:
        nxt = int(torch.argmax(forward_logits(cfg, w, toks)[-1]))
        if nxt in stop_ids:
            break
        out.append(nxt)
        toks.append(nxt)
    return out
