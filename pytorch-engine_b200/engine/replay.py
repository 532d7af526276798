"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: it builds the same
``Engine`` that generation uses and calls its step function.  Input: one JSON object per line,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries`` gives each request's next tokens and the positions among them whose logits are wanted;
a request gets a cache slot at its first appearance and gives it back when ``end`` names it.  For a
step in which something is wanted, ``<out>/<step>.f32`` holds the logits as little-endian float32
``[wanted, vocab]`` in the order of the entries and of ``want``.  After every step a line
``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import json
import os
import sys
from typing import Dict, IO, Optional

import numpy as np

from .batch import StepEntry
from .engine import Engine


class TraceError(ValueError):
    pass


class TraceReplayer:
    def __init__(self, engine: Engine, out_dir: str) -> None:
        self.engine = engine
        self.out_dir = out_dir
        os.makedirs(out_dir, exist_ok=True)
        self.slots: Dict[str, int] = {}

    def run_step(self, record: dict) -> Optional[str]:
        """Run one step record; returns the path of the logits file if one was written."""
        if "step" not in record or "entries" not in record:
            raise TraceError("a step needs the keys 'step' and 'entries'")
        step = record["step"]
        entries = []
        for e in record["entries"]:
            rid = str(e["id"])
            tokens = [int(t) for t in e["tokens"]]
            if not tokens:
                raise TraceError(f"step {step}: request {rid!r} brings no tokens")
            if rid not in self.slots:
                self.slots[rid] = self.engine.alloc_slot()
            entries.append(StepEntry(self.slots[rid], tokens, tuple(int(w) for w in e.get("want", ()))))
        written = None
        if entries:
            logits = self.engine.step(entries)
            if logits.shape[0] > 0:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                written = os.path.join(self.out_dir, f"{step}.f32")
                tmp = written + ".tmp"
                with open(tmp, "wb") as fh:
                    fh.write(np.ascontiguousarray(arr).tobytes())
                os.replace(tmp, written)
        for rid in record.get("end", ()):
            rid = str(rid)
            if rid not in self.slots:
                raise TraceError(f"step {step}: 'end' names request {rid!r}, which is not live")
            self.engine.free_slot(self.slots.pop(rid))
        return written

    def run(self, lines: IO[str], out: IO[str] = sys.stdout) -> int:
        for line in lines:
            line = line.strip()
            if not line:
                continue
            record = json.loads(line)
            self.run_step(record)
            out.write(f"done {record['step']}\n")
            out.flush()
        return 0


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(prog="trace_run", description="Feed token ids through the model step by step and write logits")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time, each request rounded up to 64")
    args = ap.parse_args(argv)
    from ..cache import PAGE_TOKENS, pages_for
    from ..config.registry import load_config

    cfg = load_config(args.model)
    cache_tokens = pages_for(max(args.max_tokens, 1)) * PAGE_TOKENS
    engine = Engine(args.model, dtype=args.dtype, max_context_len=min(cfg.max_positions, cache_tokens),
                    max_cache_tokens=cache_tokens, max_slots=min(pages_for(cache_tokens), 8192))
    return TraceReplayer(engine, args.out).run(sys.stdin)
