"""The engine against the plain implementation at a Qwen3 size, with random weights.

    python tests/parity_at_size.py --preset qwen3_0_6b
    python tests/parity_at_size.py --preset qwen3_8b --layers 4
    python tests/parity_at_size.py --preset qwen3_8b            # all 36 layers: about 70 GB on the device

For float32 and bfloat16 it replays two requests of unequal lengths through the engine's own replayer
in three ways (each alone and whole; alone with the last tokens one by one; together in one batch whose
shorter request ends earlier) and compares the logits at a spread of positions with the plain
implementation (``plain_qwen3.py``, on the CPU, the same weights).  It prints the worst error of each
way relative to the largest logit, and exits with 1 if one exceeds its limit.  The limit is the tests'
tolerance; for bfloat16 it is the larger of that and the rounding noise at this depth, measured as the
difference between the plain implementation storing its activations in bfloat16 and the same in float32:
two bfloat16 evaluations that round at the same places cannot be asked to agree better with each other
than either agrees with exact arithmetic (a flipped rounding early on is carried through every later
layer).  The tolerance alone was set for models of one to three layers.
``run()`` is what ``test_sizes_gpu.py`` calls.
"""
import argparse
import os
import sys
import tempfile
import time

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
for p in (HERE, os.path.dirname(HERE)):
    if p not in sys.path:
        sys.path.insert(0, p)

import plain_qwen3 as plain  # noqa: E402
from conftest import TOL  # noqa: E402


def _tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def _rows(path, n, vocab):
    return torch.frombuffer(bytearray(open(path, "rb").read()), dtype=torch.float32).view(n, vocab)


def run(preset: str, layers=None, lengths=(96, 41), one_by_one: int = 8, seed: int = 0, verbose: bool = True,
        **overrides):
    """{(dtype, way): worst relative error}.  ``overrides`` replace keys of the preset (a smaller vocabulary keeps
    the plain implementation's time down when the prompt is long)."""
    import pytorch_engine_b200 as pe
    from importlib import import_module

    over = dict(overrides)
    if layers:
        over["num_hidden_layers"] = int(layers)
    cfg = pe.config.preset(preset, **over)
    plan = import_module("pytorch-engine_b200.config.registry").architecture(cfg.architecture).plan(cfg)
    t0 = time.time()
    weights = import_module("pytorch-engine_b200.weights.random_init").random_weights(plan, seed, device="cuda:0")
    host = {name: t.to(torch.float32).cpu() for name, t in weights.items()}
    cfg_dict = cfg.to_dict()
    prompts = [_tokens(cfg.vocab_size, n, 100 + i) for i, n in enumerate(lengths)]
    want = [sorted({0, 1, n // 2, n - one_by_one - 1, *range(n - one_by_one, n)}) for n in lengths]
    if verbose:
        print(f"{preset}: {cfg.num_hidden_layers} layers, hidden {cfg.hidden_size}, vocabulary {cfg.vocab_size}; "
              f"weights made in {time.time() - t0:.1f} s", flush=True)
    worst = {}
    exact = None
    for dtype in ("float32", "bfloat16"):
        t0 = time.time()
        store = torch.bfloat16 if dtype == "bfloat16" else None
        refs = [plain.forward_logits(cfg_dict, host, p, store=store) for p in prompts]
        scale = max(float(r.abs().max()) for r in refs)
        t_plain = time.time() - t0
        if dtype == "float32":
            exact = refs
        else:
            worst[dtype, NOISE] = max(
                float((a.double() - b.double()).abs().max()) for a, b in zip(refs, exact)) / scale
        eng = pe.Engine(None, config=cfg, weights=dict(weights), dtype=dtype, max_context_len=max(256, max(lengths) + 64),
                        max_cache_tokens=max(1024, 4 * (sum(lengths) + 128)), max_batch=4)
        with tempfile.TemporaryDirectory() as out:
            rep = pe.engine.replay.TraceReplayer(eng, out)
            step = [0]

            def feed(entries, end=()):
                rec = {"step": step[0], "entries": [{"id": i, "tokens": t, "want": w} for i, t, w in entries],
                       "end": list(end)}
                step[0] += 1
                path = rep.run_step(rec)
                n = sum(len(w) for _, _, w in entries)
                return _rows(path, n, cfg.vocab_size) if n else None

            def err(rows, ref_rows):
                return float((rows.double() - ref_rows.double()).abs().max()) / scale

            e = 0.0
            for r, (p, w) in enumerate(zip(prompts, want)):
                e = max(e, err(feed([(f"w{r}", p, w)], end=[f"w{r}"]), refs[r][w]))
            worst[dtype, "whole"] = e
            e = 0.0
            for r, p in enumerate(prompts):
                n = len(p)
                head = [i for i in want[r] if i < n - one_by_one]
                e = max(e, err(feed([(f"o{r}", p[:n - one_by_one], head)]), refs[r][head]))
                for i in range(n - one_by_one, n):
                    e = max(e, err(feed([(f"o{r}", [p[i]], [0])], end=[f"o{r}"] if i == n - 1 else []), refs[r][[i]]))
            worst[dtype, "last tokens one by one"] = e
            # both together: prompts without their last tokens in one step, then one token each; the shorter ends first
            cut = [len(p) - one_by_one for p in prompts]
            heads = [[i for i in w if i < c] for w, c in zip(want, cut)]
            rows = feed([(f"b{r}", p[:c], h) for r, (p, c, h) in enumerate(zip(prompts, cut, heads))])
            e = err(rows, torch.cat([refs[r][h] for r, h in enumerate(heads)]))
            short = min(range(len(prompts)), key=lambda r: len(prompts[r]))
            for j in range(one_by_one):
                live = [r for r in range(len(prompts)) if not (r == short and j >= one_by_one // 2)]
                ends = [f"b{short}"] if j == one_by_one // 2 - 1 else ([f"b{r}" for r in live] if j == one_by_one - 1 else [])
                rows = feed([(f"b{r}", [prompts[r][cut[r] + j]], [0]) for r in live], end=ends)
                e = max(e, err(rows, torch.cat([refs[r][[cut[r] + j]] for r in live])))
            worst[dtype, "unequal batch"] = e
        assert not eng.cache.live_slots
        del eng, rep
        torch.cuda.empty_cache()
        if verbose:
            for (d, way), v in worst.items():
                if d == dtype:
                    print(f"  {dtype:8s} {way:46s} {v:.2e} of the largest logit (limit {limit(worst, dtype):.1e})", flush=True)
            print(f"  ({dtype}: plain implementation {t_plain:.1f} s, engine and replay {time.time() - t0 - t_plain:.1f} s)",
                  flush=True)
    return worst


NOISE = "rounding noise of the plain implementation"


def limit(worst, dtype: str) -> float:
    return max(TOL[dtype], worst.get((dtype, NOISE), 0.0))


def failures(worst):
    return {k: v for k, v in worst.items() if k[1] != NOISE and not v < limit(worst, k[0])}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="qwen3_0_6b")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the preset has")
    ap.add_argument("--lengths", default="96,41")
    ap.add_argument("--vocab", type=int, default=None, help="another vocabulary size than the preset's")
    a = ap.parse_args()
    worst = run(a.preset, a.layers, tuple(int(x) for x in a.lengths.split(",")),
                **({"vocab_size": a.vocab} if a.vocab else {}))
    bad = failures(worst)
    print("parity " + ("FAILED: " + str(bad) if bad else "ok"))
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
