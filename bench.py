#!/usr/bin/env python3
"""Benchmark: decode tokens/s of a Qwen3-8B-shaped model (random weights, bfloat16) on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --micro gemm|gemm_mid|prefill_attention|decode_attention|rope_append|sampler   (single kernels, text)

A step is one decode step: every live sequence gets one token (model step + sampler).  The default
run has the layer sizes of the Qwen3-8B shape, a batch of 8 and a context of 4,096.  One JSON line
is printed: ``value`` is decoded tokens/s timed on the device with CUDA events; ``e2e`` is the same
through the Python entry point (``Engine.stream_tokens``: host token ids in, host token ids out
every step; untimed decode steps after the prompts (at least 48: the clocks need them after a whole
batch of prompts), then K timed ones, with per-step host times and the clocks seen); ``prefill`` is
one 2,048-token prompt; ``roofline`` is the bytes a decode step must read (every weight once, the
cache of the live requests) over its time; ``points`` holds decode at batch 1 and 64; ``baseline``
and ``vs_baseline`` come from a plain PyTorch model of the same shape timed on the same GPU
(baseline/plain_torch.py).  For the device-timed decode numbers the cache is brought to the wanted
length by reserving pages over storage filled with random values (what a decode step costs does not
depend on the values); the end-to-end number runs real prompts through the public API.
``--impl reference`` runs the unmodified reference instead (baseline/reference_arm.py: its own
engine on an F16 GGUF of the same shape, the requests one after another) and prints the same keys.
"""
import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

E2E_MIN_WARMUP = 48    # untimed decode steps between the prompts and the timed steps of the end-to-end figure

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as fh:
                d = json.load(fh)
            hbm = d.get("hbm_gbs")
            tf = d.get("bf16_tflops")
            if hbm and tf:
                return {"hbm_gbs": float(hbm), "bf16_tflops": float(tf),
                        "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", tf)), "source": "measured"}
        except Exception:
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "25"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.rows.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def model_numbers(cfg, layers):
    """Parameter counts and per-token cache bytes from the configuration (bfloat16 storage)."""
    h, nh, nkv, d, inter, v = (cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                               cfg.intermediate_size, cfg.vocab_size)
    per_layer = (nh + 2 * nkv) * d * h + nh * d * h + 3 * inter * h
    return {
        "linear_params_per_layer": per_layer,
        "head_params": v * h,
        "norm_params": layers * (2 * h + 2 * d) + h,
        "kv_bytes_per_token": layers * 2 * nkv * d * 2,
        "attn_flops_per_layer": lambda t: 2 * nh * d * t * t,
    }


def decode_bytes(cfg, layers, batch, mean_len):
    n = model_numbers(cfg, layers)
    weights = (layers * n["linear_params_per_layer"] + n["head_params"]) * 2 + n["norm_params"] * 4
    return weights + batch * cfg.hidden_size * 2 + batch * mean_len * n["kv_bytes_per_token"]


def prefill_flops(cfg, layers, tokens):
    n = model_numbers(cfg, layers)
    return 2 * tokens * layers * n["linear_params_per_layer"] + layers * n["attn_flops_per_layer"](tokens) + 2 * n["head_params"]


def reference_arm(args):
    """``--impl reference``: the unmodified reference through its own public API (baseline/reference_arm.py,
    which imports nothing of this repository's package), same metric, same sizes, same JSON keys."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import reference_arm as arm

        with open(os.path.join(ROOT, "pytorch-engine_b200", "config", "presets", args.preset + ".json")) as fh:
            cfg = json.load(fh)
        import contextlib
        with contextlib.redirect_stdout(sys.stderr):     # the reference prints its progress to standard output
            out = arm.run(cfg, preset_name=args.preset, batch=args.batch, context=args.context, steps=args.steps,
                          warmup=args.warmup, layers=args.layers)
    except BaseException as exc:  # the arm says why it cannot run; it never fails the benchmark
        if isinstance(exc, KeyboardInterrupt):
            raise
        text = str(exc).strip().splitlines()
        out = {"impl": "reference", "unavailable": f"{type(exc).__name__}: {text[0][:300] if text else ''}"}
    print(json.dumps(out))
    return 0


def plain_torch_baseline(cfg_dict, layers, args):
    """The plain PyTorch model of the same shape on the same GPU (baseline/plain_torch.py: library calls only)."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import plain_torch

    return plain_torch.measure(cfg_dict, layers, context=args.context, batches=sorted({1, args.batch, 64}),
                               prefill_tokens=0 if args.no_prefill else args.prefill_tokens)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--preset", type=str, default="qwen3_8b")
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the preset has (named in config)")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-points", action="store_true")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--no-cuda-graph", action="store_true")
    ap.add_argument("--no-baseline", action="store_true", help="skip the plain PyTorch model that vs_baseline divides by")
    ap.add_argument("--micro", type=str, default=None,
                    help="time single kernels at the preset's sizes instead (gemm, prefill_attention, decode_attention, rope_append, sampler) and print text")
    args = ap.parse_args()

    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return reference_arm(args)

    import torch

    pe = importlib.import_module("pytorch-engine_b200")
    ops = pe.kernels.ops
    if args.micro:
        import bench_micro as micro
        if args.micro not in micro.CASES:
            print(f"bench.py: --micro takes one of {sorted(micro.CASES)}")
            return 2
        micro.CASES[args.micro](pe.preset(args.preset), "cuda:0")
        return 0
    peaks = load_peaks()
    full = pe.preset(args.preset)
    layers_model = full.num_hidden_layers
    cfg = pe.preset(args.preset, num_hidden_layers=args.layers) if args.layers else full
    layers = cfg.num_hidden_layers
    B, ctx, K, W = args.batch, args.context, args.steps, args.warmup
    max_b = max(B, 64 if not args.no_points else B)
    t_load = time.perf_counter()
    # the cache holds whole pages of 64 tokens: a context that is no multiple of 64 still takes its last page
    engine = pe.Engine.from_random(cfg, seed=0, dtype="bfloat16", max_context_len=ctx, max_cache_tokens=max_b * (-(-ctx // 64) * 64),
                                   max_batch=max_b, enable_cuda_graph=not args.no_cuda_graph)
    for g in engine.cache.groups:
        if g.storage is not None:
            g.storage.normal_(0.0, 0.5)
    torch.cuda.synchronize()
    load_s = time.perf_counter() - t_load
    gen = torch.Generator().manual_seed(1)
    vocab = cfg.vocab_size
    greedy = pe.SamplingParams.greedy_params(max_tokens=1)

    def measure_decode(batch, steps, warmup, sample_clocks=False):
        """ms per decode step at `batch`, the last timed step ending at context `ctx`."""
        start_len = ctx - steps - warmup
        slots = [engine.alloc_slot() for _ in range(batch)]
        for s in slots:
            engine.cache.reserve(s, start_len)
            engine.cache.commit(s, start_len)
        toks = torch.randint(0, vocab, (steps + warmup, batch), generator=gen).tolist()
        reqs = list(range(batch))
        # the sampler as the engine runs it: rows cut into chunks by a first kernel (it needs a scratch)
        need = ops.sample_scratch_bytes(batch, vocab, 0.0, 0, 1.0, 0.0)
        scratch = torch.empty(need, dtype=torch.uint8, device=engine.device) if need else None

        def one(i):
            logits = engine.runner.step([pe.StepEntry(s, (toks[i][j],), (0,)) for j, s in enumerate(slots)], check=False)
            meta = torch.tensor([reqs, [i] * batch], dtype=torch.int32).to(engine.device, non_blocking=True)
            out = torch.empty((batch,), dtype=torch.int32, device=engine.device)
            ops.sample(logits, 0.0, 0, 1.0, 0.0, 0, meta[0], meta[1], out, scratch=scratch)
            return out

        for i in range(warmup):
            one(i)
        torch.cuda.synchronize()
        sampler = ClockSampler() if sample_clocks else None
        if sampler:
            sampler.start()
            time.sleep(0.25)
        launches0 = ops.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for i in range(warmup, warmup + steps):
            one(i)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        launches = ops.launch_count() - launches0
        clocks = sampler.stop() if sampler else None
        engine.runtime.raise_on_status()
        for s in slots:
            engine.free_slot(s)
        mean_len = start_len + warmup + (steps + 1) / 2.0
        return ms, launches, clocks, mean_len

    ms, launches, clocks, mean_len = measure_decode(B, K, W, sample_clocks=True)
    value = B * 1000.0 / ms
    bytes_step = decode_bytes(cfg, layers, B, mean_len)
    achieved = bytes_step / (ms * 1e-3) / 1e9
    out = {
        "metric": f"{args.preset}_shape_bf16_decode_tokens_per_s_batch{B}_ctx{ctx}",
        "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {
            "model": f"{args.preset} shape, random weights N(0,0.02), seed 0", "layers": layers,
            "layers_in_model": layers_model, "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
            "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size,
            "vocab": cfg.vocab_size, "global_batch": B, "seq_len": ctx, "prefill_tokens": args.prefill_tokens,
            "parallelism": "single-gpu", "cuda_graph": not args.no_cuda_graph,
            "l2": "inputs larger than L2 (weights read every step exceed 126 MB)",
            "cache": "paged bf16, random fill for device-timed decode", "peaks": peaks["source"],
        },
        "clocks": clocks, "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "bytes_per_step": int(bytes_step)},
        "load_s": round(load_s, 1),
    }

    if not args.no_prefill:
        T = args.prefill_tokens
        times = []
        for it in range(7):   # the first is warm-up
            s = engine.alloc_slot()
            toks = torch.randint(0, vocab, (T,), generator=gen).tolist()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            engine.runner.step([pe.StepEntry(s, toks, (T - 1,))], check=False)
            e1.record()
            torch.cuda.synchronize()
            if it > 0:
                times.append(e0.elapsed_time(e1))
            engine.free_slot(s)
        pms = statistics.median(times)
        fl = prefill_flops(cfg, layers, T)
        out["prefill"] = {"value": round(T * 1000.0 / pms, 1), "tokens": T, "ms": round(pms, 3),
                          "frac": round(fl / (pms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4), "flops": int(fl),
                          # frac is against the library product's burst figure; the same against what it holds
                          # for seconds under the power cap, which a 26 ms step of products already runs into
                          "frac_of_sustained": round(fl / (pms * 1e-3) / (peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]) * 1e12), 4)}

    if not args.no_points:
        pts = {}
        for b in (1, 64):
            pms, _, _, _ = measure_decode(b, max(8, min(K, 32)), 4)
            pts[f"decode_b{b}"] = round(b * 1000.0 / pms, 2)
        out["points"] = pts

    if not args.no_e2e:
        # through the public API: real prompts, host token ids in and out at every step.  The prompts of a
        # whole batch are seconds' worth of tensor-core work at the board's power cap, after which the clocks
        # come back over some tens of decode steps; so the untimed steps before the K timed ones are at least
        # E2E_MIN_WARMUP (the device-timed figure above never sees a prefill).  Host time stamps of every step
        # and the SM clock sampled meanwhile are kept, so that what the clocks cost can be read off the line.
        steps_e = max(8, K)
        warm_e = max(W, E2E_MIN_WARMUP)
        plen = ctx - steps_e - warm_e - 1
        prompts = [torch.randint(0, vocab, (plen,), generator=gen).tolist() for _ in range(B)]
        params = pe.SamplingParams.greedy_params(max_tokens=steps_e + warm_e + 1)
        got = [0] * B
        stamps = []                      # host time at which every request has its k-th token
        sampler = ClockSampler()
        sampler.start()
        t_begin = time.perf_counter()
        for chunk in engine.stream_tokens(prompts, params):
            got[chunk.request] += 1
            if min(got) > len(stamps):
                stamps.append(time.perf_counter())
        torch.cuda.synchronize()
        clocks_e = sampler.stop()
        # stamps[0]: first tokens (end of the prompts); stamps[warm_e]: W untimed steps later; then K timed steps
        dt = stamps[warm_e + steps_e] - stamps[warm_e]
        n_tokens = B * steps_e
        step_ms = [(b - a) * 1e3 for a, b in zip(stamps[:-1], stamps[1:])]
        out["e2e"] = {"value": round(n_tokens / dt, 2), "unit": "tokens/s", "tokens": n_tokens,
                      "h2d_bytes_per_step": (B + 3 * B + 1 + B) * 4 + 2 * B * 4, "d2h_bytes_per_step": B * 4 + 16,
                      "ms_per_step": round(dt * 1e3 / steps_e, 4),
                      "prompt_s": round(stamps[0] - t_begin, 3),
                      "ms_first_steps_after_prompts": [round(x, 2) for x in step_ms[:4]],
                      "ms_per_step_untimed": round(sum(step_ms[:warm_e]) / warm_e, 4),
                      "sm_mhz_median_whole_run": clocks_e.get("sm_mhz"), "clock_reasons": clocks_e.get("reasons"),
                      "api": "Engine.stream_tokens, greedy, prompts of %d tokens, %d untimed steps, %d timed" % (plen, warm_e, steps_e)}

    if not args.no_baseline:
        # the same shape as a plain PyTorch model (library products and attention, eager) on this GPU
        base = plain_torch_baseline(cfg.to_dict(), layers, args)
        out["baseline"] = {"what": "plain PyTorch (F.linear bf16, scaled_dot_product_attention, eager, contiguous cache), same GPU"}
        for k, v in base.items():
            out["baseline"][k] = v["tokens_per_s"]
        mine = base.get(f"decode_b{B}")
        if mine:
            out["vs_baseline"] = round(value / mine["tokens_per_s"], 3)
            out["baseline"]["ms_per_step"] = mine["ms_per_step"]

    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
