#!/usr/bin/env python3
"""The reference arm of the benchmark: binief/pytorch-engine itself, unmodified, through its own public API.

It imports nothing of this repository's package.  What it does:

1. finds the reference's source tree (``baseline/_ref/`` beside this file, a plain copy of the
   checkout: the project has neither ``setup.py`` nor ``pyproject.toml``, so ``pip install`` refuses it
   and its own notebooks run it from the source tree as well);
2. writes a float16 GGUF file of the wanted Qwen3 shape with random N(0, 0.02) weights using
   ``gguf.GGUFWriter`` (the technique of the reference's own fixture, tests/test_pygguf_engine.py:105-200),
   one random matrix per tensor kind reused by every layer: what a step costs does not depend on the values;
3. runs ``PyGGUFEngine(path, kv_dtype="fp16", speculative_ngram=False, speculative_mtp=False,
   max_context_len=ctx)`` and ``.stream_tokens(ids, SamplingConfig(temperature=0, cache_prompt=False))``
   (pygguf_engine/engine.py:259-291, 511-935) for ``batch`` prompts one after another, since the reference
   runs one sequence at a time (pygguf_engine/kv_cache.py:1877): that is its stock path for several requests;
4. reports decoded tokens per second over all the requests: W untimed decoded tokens per request, then K
   timed ones, the timed region of each request bracketed by CUDA events (``value``) and by the host
   clock around the tokens as the API hands them over (``e2e``).

Its linears run in float16 (pygguf_engine/quant_kernels.py:1807-1809, 1836), the reference's only
unquantised precision; bfloat16 does not exist there.
"""
from __future__ import annotations

import json
import os
import shutil
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))


def find_reference():
    for cand in (os.path.join(HERE, "_ref"), os.environ.get("PE_B200_REFERENCE", "")):
        if cand and os.path.isfile(os.path.join(cand, "pygguf_engine", "engine.py")):
            return cand
    return None


def write_random_gguf(path, cfg, layers, seed=0):
    """A float16 GGUF of the Qwen3 shape ``cfg`` (config.json keys) with ``layers`` blocks."""
    import gguf
    import numpy as np

    rng = np.random.default_rng(seed)
    h, nh, nkv, d = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    inter, vocab = cfg["intermediate_size"], cfg["vocab_size"]

    def matrix(rows, cols):
        out = np.empty((rows, cols), dtype=np.float16)
        step = max(1, (1 << 24) // cols)
        for r in range(0, rows, step):
            n = min(step, rows - r)
            out[r:r + n] = (rng.standard_normal((n, cols), dtype=np.float32) * 0.02).astype(np.float16)
        return out

    def norm(n):
        return (1.0 + 0.02 * rng.standard_normal(n, dtype=np.float32)).astype(np.float32)

    w = gguf.GGUFWriter(path, "qwen3")
    w.add_name("random-qwen3")
    w.add_block_count(layers)
    w.add_embedding_length(h)
    w.add_feed_forward_length(inter)
    w.add_head_count(nh)
    w.add_head_count_kv(nkv)
    w.add_key_length(d)
    w.add_value_length(d)
    w.add_context_length(cfg["max_position_embeddings"])
    w.add_layer_norm_rms_eps(cfg["rms_norm_eps"])
    w.add_rope_dimension_count(d)
    w.add_rope_freq_base(cfg["rope_theta"])
    w.add_tokenizer_model("gpt2")
    w.add_token_list([f"tok_{i}" for i in range(vocab)])
    w.add_eos_token_id(vocab - 1)
    w.add_tensor("token_embd.weight", matrix(vocab, h))
    per_layer = {
        "attn_q.weight": matrix(nh * d, h), "attn_k.weight": matrix(nkv * d, h), "attn_v.weight": matrix(nkv * d, h),
        "attn_output.weight": matrix(h, nh * d), "ffn_gate.weight": matrix(inter, h), "ffn_up.weight": matrix(inter, h),
        "ffn_down.weight": matrix(h, inter), "attn_norm.weight": norm(h), "ffn_norm.weight": norm(h),
        "attn_q_norm.weight": norm(d), "attn_k_norm.weight": norm(d),
    }
    for i in range(layers):
        for name, arr in per_layer.items():
            w.add_tensor(f"blk.{i}.{name}", arr)
    w.add_tensor("output_norm.weight", norm(h))
    if not cfg.get("tie_word_embeddings", False):
        w.add_tensor("output.weight", matrix(vocab, h))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


def gguf_bytes(cfg, layers):
    h, nh, nkv, d = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    inter, vocab = cfg["intermediate_size"], cfg["vocab_size"]
    per_layer = (nh + 2 * nkv) * d * h + nh * d * h + 3 * inter * h
    heads = (1 if cfg.get("tie_word_embeddings", False) else 2) * vocab * h
    return 2 * (layers * per_layer + heads)


def run(cfg, *, preset_name, batch, context, steps, warmup, layers=None, device="cuda:0", scratch_dir=None, log=None):
    """Runs the arm; returns the dict that ``bench.py --impl reference`` prints."""
    say = log or (lambda m: print(f"[reference arm] {m}", file=sys.stderr, flush=True))
    ref = find_reference()
    if ref is None:
        return {"impl": "reference", "unavailable": "no copy of the reference's source tree under baseline/_ref"}
    layers_model = cfg["num_hidden_layers"]
    asked = layers = layers or layers_model
    base = scratch_dir or tempfile.gettempdir()
    need = gguf_bytes(cfg, layers) + (1 << 30)
    free = shutil.disk_usage(base).free
    while layers > 1 and gguf_bytes(cfg, layers) + (1 << 30) > free:
        layers = max(1, layers // 2)          # a scratch disk too small for the whole file: fewer layers, and said so
    if layers != asked:
        say(f"scratch folder {base} has {free / 1e9:.1f} GB free, the file needs {need / 1e9:.1f}: writing {layers} layers")
    sys.path.insert(0, ref)
    import torch

    tmp = tempfile.mkdtemp(prefix="pe_b200_refarm_", dir=base)
    try:
        path = os.path.join(tmp, "model.gguf")
        t0 = time.perf_counter()
        write_random_gguf(path, cfg, layers)
        say(f"wrote {os.path.getsize(path) / 1e9:.2f} GB GGUF ({layers} layers) in {time.perf_counter() - t0:.0f} s")
        from pygguf_engine.engine import PyGGUFEngine, SamplingConfig

        t0 = time.perf_counter()
        engine = PyGGUFEngine(path, kv_dtype="fp16", devices=[device], speculative_ngram=False, speculative_mtp=False,
                              max_context_len=context)
        load_s = time.perf_counter() - t0
        cuda = device.startswith("cuda")
        gen = torch.Generator().manual_seed(1)
        vocab = cfg["vocab_size"]
        new_tokens = steps + warmup + 1
        plen = context - new_tokens
        dev_ms = 0.0
        host_s = 0.0
        timed_tokens = 0
        prefill_s = []
        stats_decode = []
        for r in range(batch):
            ids = torch.randint(0, vocab - 1, (plen,), generator=gen).tolist()
            sampling = SamplingConfig(max_tokens=new_tokens, temperature=0.0, cache_prompt=False)
            got = 0
            e0 = e1 = None
            t_first = None
            t_start = time.perf_counter()
            for chunk in engine.stream_tokens(ids, sampling):
                if chunk.stats is not None:
                    stats_decode.append((chunk.stats.completion_tokens, chunk.stats.decode_time_s))
                    prefill_s.append(chunk.stats.prefill_time_s)
                if chunk.finish_reason == "stop":
                    break                      # the closing chunk of a stopped request repeats its last token
                got += 1
                if got == warmup + 1:
                    t_first = time.perf_counter()
                    if cuda:
                        e0 = torch.cuda.Event(enable_timing=True)
                        e0.record()
                if chunk.finish_reason is not None:
                    break
            if cuda:
                e1 = torch.cuda.Event(enable_timing=True)
                e1.record()
                torch.cuda.synchronize()
            t_end = time.perf_counter()
            if t_first is None or got <= warmup + 1:
                say(f"request {r}: ended after {got} tokens, before the timed region")
                continue
            n = got - (warmup + 1)
            timed_tokens += n
            host_s += t_end - t_first
            dev_ms += e0.elapsed_time(e1) if cuda else (t_end - t_first) * 1e3
            say(f"request {r}: prompt {plen} tokens in {t_first - t_start:.2f} s to token {warmup + 1}; "
                f"{n} timed tokens in {t_end - t_first:.3f} s")
        if timed_tokens == 0:
            return {"impl": "reference", "unavailable": "every request ended before the timed region (stop token)"}
        ms_per_token = dev_ms / timed_tokens
        value = 1000.0 / ms_per_token
        out = {
            "metric": f"{preset_name}_shape_decode_tokens_per_s_batch{batch}_ctx{context}",
            "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
            "ms_per_step": round(ms_per_token * batch, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp16", "data": "synthetic", "impl": "reference",
            "config": {
                "model": f"{preset_name} shape, random weights N(0,0.02) as an F16 GGUF", "layers": layers,
                "layers_in_model": layers_model, "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                "intermediate": cfg["intermediate_size"], "vocab": vocab, "global_batch": batch, "seq_len": context,
                "parallelism": "single-gpu", "batching": "none in the reference: the requests run one after another",
                "api": "PyGGUFEngine.stream_tokens, temperature 0, kv fp16, no speculation, its own CUDA graphs",
                "l2": "inputs larger than L2 (weights read every token exceed 126 MB)",
            },
            "e2e": {"value": round(timed_tokens / host_s, 2), "unit": "tokens/s", "tokens": timed_tokens,
                    "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 8},
            "gpu_launches": None,
            "prefill": {"tokens": plen, "ms": round(1e3 * sorted(prefill_s)[len(prefill_s) // 2], 2),
                        "value": round(plen / sorted(prefill_s)[len(prefill_s) // 2], 1)} if prefill_s else None,
            "own_stats_decode_tokens_per_s": round(sum(n for n, _ in stats_decode) / max(1e-9, sum(s for _, s in stats_decode)), 2),
            "load_s": round(load_s, 1),
        }
        return out
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


def main():
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True, help="a config.json of the shape to run")
    ap.add_argument("--name", default="custom")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args()
    with open(args.config) as fh:
        cfg = json.load(fh)
    try:
        out = run(cfg, preset_name=args.name, batch=args.batch, context=args.context, steps=args.steps,
                  warmup=args.warmup, layers=args.layers, device=args.device)
    except Exception as exc:  # the arm reports why it cannot run instead of failing the benchmark
        out = {"impl": "reference", "unavailable": f"{type(exc).__name__}: {str(exc).splitlines()[0][:300] if str(exc) else ''}"}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
