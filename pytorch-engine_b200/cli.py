"""Command line: generate from token ids with a model folder or a random model.

    python -m pytorch-engine_b200.cli --model DIR --prompt-ids 1,2,3 --max-tokens 16 --temperature 0

The reference's command line starts a server (kaggle_serve.py:292-383); its flags that concern the
engine keep their names and meanings here (``--ctx``, ``--no-cuda-graph``), ``--gguf`` becomes
``--model`` (a folder with config.json and safetensors), and the per-request options of its
``SamplingConfig`` (pygguf_engine/engine.py:28-45) are flags of their own.
"""
from __future__ import annotations

import argparse
import json
import random
import sys
from typing import List


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="pytorch-engine_b200", description="Generate tokens on one B200 from a model folder or a random model of a named size")
    src = p.add_argument_group("model")
    src.add_argument("--model", type=str, default=None, help="folder with config.json and model.safetensors")
    src.add_argument("--random", type=str, default=None, metavar="PRESET",
                     help="random weights for a named size (see --list-presets) instead of --model")
    src.add_argument("--seed", type=int, default=0, help="seed of the random weights")
    src.add_argument("--write-random", type=str, default=None, metavar="DIR",
                     help="write the random model (config.json + model.safetensors) to DIR and exit")
    src.add_argument("--list-presets", action="store_true")
    p.add_argument("--dtype", choices=["bf16", "bfloat16", "fp32", "float32"], default="bf16")
    p.add_argument("--ctx", type=int, default=None, help="max context window (default: the model's)")
    p.add_argument("--max-batch", type=int, default=64, help="most sequences decoded together")
    p.add_argument("--max-step-tokens", type=int, default=65536, help="most prompt tokens fed in one step (0: no limit)")
    p.add_argument("--no-cuda-graph", action="store_true", help="disable CUDA graph replay of decode steps")
    pr = p.add_argument_group("prompts (token ids)")
    pr.add_argument("--prompt-ids", action="append", default=[], metavar="1,2,3", help="a prompt as token ids; repeatable")
    pr.add_argument("--prompt-file", type=str, default=None, help="file with one prompt per line (comma or space separated ids)")
    pr.add_argument("--random-prompts", type=str, default=None, metavar="LEN[,LEN...]",
                    help="uniform-random prompts of these lengths")
    pr.add_argument("--prompt", action="append", default=[], metavar="TEXT",
                    help="a prompt as text; needs tokenizer.json in the model folder (repeatable)")
    sm = p.add_argument_group("sampling")
    sm.add_argument("--max-tokens", type=int, default=512)
    sm.add_argument("--temperature", type=float, default=0.7)
    sm.add_argument("--top-k", type=int, default=40)
    sm.add_argument("--top-p", type=float, default=0.95)
    sm.add_argument("--min-p", type=float, default=0.05)
    sm.add_argument("--repetition-penalty", type=float, default=1.0)
    sm.add_argument("--sampling-seed", type=int, default=None)
    sm.add_argument("--stop-token-ids", type=str, default="", metavar="1,2")
    p.add_argument("--json", action="store_true", help="print one JSON line per request instead of text")
    return p


def _ids(text: str) -> List[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def load_tokenizer(model_dir):
    """The folder's ``tokenizer.json`` as a ``tokenizers.Tokenizer``, or None (no folder, no file, no package).
    The engine itself works on token ids only; this is a convenience of the command line."""
    import os

    if not model_dir or not os.path.isfile(os.path.join(model_dir, "tokenizer.json")):
        return None
    try:
        from tokenizers import Tokenizer
    except ImportError:
        return None
    return Tokenizer.from_file(os.path.join(model_dir, "tokenizer.json"))


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    from . import Engine, SamplingParams, load_config, preset, write_random_model
    from .config import preset_names

    if args.list_presets:
        print("\n".join(preset_names()))
        return 0
    if (args.model is None) == (args.random is None):
        print("give exactly one of --model DIR or --random PRESET", file=sys.stderr)
        return 2
    if args.write_random:
        if args.random is None:
            print("--write-random needs --random PRESET", file=sys.stderr)
            return 2
        write_random_model(args.write_random, preset(args.random), args.seed)
        print(f"wrote {args.write_random}")
        return 0
    cfg = load_config(args.model) if args.model else preset(args.random)
    prompts: List[List[int]] = [_ids(t) for t in args.prompt_ids]
    if args.prompt_file:
        with open(args.prompt_file) as fh:
            prompts += [_ids(line) for line in fh if line.strip()]
    if args.random_prompts:
        rng = random.Random(args.seed)
        vocab = getattr(cfg, "vocab_size")
        prompts += [[rng.randrange(vocab) for _ in range(n)] for n in _ids(args.random_prompts)]
    tokenizer = None
    if args.prompt:
        tokenizer = load_tokenizer(args.model)
        if tokenizer is None:
            print("--prompt TEXT needs --model DIR with a tokenizer.json in it (and the `tokenizers` package); "
                  "give token ids with --prompt-ids otherwise", file=sys.stderr)
            return 2
        prompts += [list(tokenizer.encode(text).ids) for text in args.prompt]
    if not prompts:
        print("no prompt given (--prompt-ids, --prompt-file, --random-prompts or --prompt)", file=sys.stderr)
        return 2
    kw = dict(dtype=args.dtype, max_context_len=args.ctx, max_batch=args.max_batch,
              max_step_tokens=args.max_step_tokens or None,
              enable_cuda_graph=not args.no_cuda_graph, verbose=not args.json)
    engine = Engine(args.model, **kw) if args.model else Engine.from_random(cfg, args.seed, **kw)
    params = SamplingParams(max_tokens=args.max_tokens, temperature=args.temperature, top_k=args.top_k,
                            top_p=args.top_p, min_p=args.min_p, repetition_penalty=args.repetition_penalty,
                            seed=args.sampling_seed, stop_token_ids=_ids(args.stop_token_ids))
    results = engine.generate(prompts, params)
    for i, r in enumerate(results):
        if args.json:
            print(json.dumps({"request": i, "token_ids": r.token_ids, "prompt_tokens": r.prompt_tokens,
                              "completion_tokens": r.completion_tokens, "finish_reason": r.finish_reason,
                              "prefill_time_s": round(r.prefill_time_s, 6), "decode_time_s": round(r.decode_time_s, 6),
                              "decode_tok_per_s": round(r.decode_tok_per_s, 2),
                              **({"text": tokenizer.decode(r.token_ids)} if tokenizer is not None else {})}))
        else:
            shown = tokenizer.decode(r.token_ids) if tokenizer is not None else " ".join(map(str, r.token_ids))
            print(f"[{i}] {r.finish_reason} after {r.completion_tokens} tokens ({r.decode_tok_per_s:.1f} tok/s): {shown}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
