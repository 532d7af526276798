"""Weights from safetensors, by tensor name.

What a model needs is read off its plan: every part declares its weights (shape and role), the
plan maps them to checkpoint tensor names.  The file set is ``model.safetensors`` or the shards
named by ``model.safetensors.index.json``.  One check compares the two sides and reports, in a
single error, every missing tensor, every unexpected tensor and every wrong shape.

Storage types: 16-bit floats are kept as bfloat16, a tensor stored in 32-bit floats stays float32,
64-bit floats become float32, integer tables become int32.  (The reference reads GGUF by name,
pygguf_engine/gguf_parser.py:236-267, floats via pygguf_engine/quant_kernels.py:1097-1116; a
missing tensor is a bare KeyError there.)
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Tuple

import torch

from ..parts.registry import lookup
from ..parts.spec import ModelPlan, WeightDecl


class WeightError(ValueError):
    """The checkpoint does not match the model; ``missing``, ``unexpected`` and ``wrong_shape`` list how."""

    def __init__(self, folder: str, missing, unexpected, wrong_shape, bad_dtype=()) -> None:
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.bad_dtype = list(bad_dtype)
        lines = [f"checkpoint in {folder!r} does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: file has {list(got)}, model wants {list(want)}" for n, got, want in self.wrong_shape))
        if self.bad_dtype:
            lines.append(f"  unusable dtypes ({len(self.bad_dtype)}): " + "; ".join(f"{n}: {dt}" for n, dt in self.bad_dtype))
        super().__init__("\n".join(lines))


def expected_tensors(plan: ModelPlan) -> Dict[str, WeightDecl]:
    """Checkpoint tensor name -> declaration, over every part of the plan.  A name used by two
    parts (tied embedding and head) must be declared with one shape."""
    out: Dict[str, WeightDecl] = {}
    for label, role, spec in plan.part_specs():
        decls = lookup(role, spec.kind).weight_decls(spec.params)
        for local, decl in decls.items():
            if local not in spec.weights:
                raise KeyError(f"{label}: the plan gives no checkpoint name for weight {local!r} of kind {spec.kind!r}")
            name = spec.weights[local]
            if name in out and tuple(out[name].shape) != tuple(decl.shape):
                raise ValueError(f"tensor {name!r} is used with two shapes: {out[name].shape} and {decl.shape}")
            out.setdefault(name, decl)
    return out


_FLOAT_KEEP = {torch.float32: torch.float32, torch.float64: torch.float32,
               torch.bfloat16: torch.bfloat16, torch.float16: torch.bfloat16}
_INT_TYPES = (torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8)


def stored_dtype(dtype: torch.dtype) -> torch.dtype:
    """The dtype a stored tensor is kept in after loading (see the module text)."""
    if dtype in _FLOAT_KEEP:
        return _FLOAT_KEEP[dtype]
    if dtype in _INT_TYPES:
        return torch.int32
    raise TypeError(str(dtype))


def _files_of(folder: str) -> List[str]:
    index = os.path.join(folder, "model.safetensors.index.json")
    single = os.path.join(folder, "model.safetensors")
    if os.path.isfile(index):
        with open(index) as fh:
            weight_map = json.load(fh).get("weight_map", {})
        return sorted({os.path.join(folder, f) for f in weight_map.values()})
    if os.path.isfile(single):
        return [single]
    raise FileNotFoundError(f"no model.safetensors (or model.safetensors.index.json) in model folder {folder!r}")


def load_weights(folder: str, plan: ModelPlan, device="cpu") -> Dict[str, torch.Tensor]:
    """{checkpoint name: tensor on ``device``} for every tensor the plan needs, after the check."""
    from safetensors import safe_open

    want = expected_tensors(plan)
    files = _files_of(folder)
    where: Dict[str, Tuple[str, Tuple[int, ...], str]] = {}
    for path in files:
        with safe_open(path, framework="pt", device="cpu") as fh:
            for name in fh.keys():
                sl = fh.get_slice(name)
                where[name] = (path, tuple(sl.get_shape()), sl.get_dtype())
    missing = sorted(n for n in want if n not in where)
    unexpected = sorted(n for n in where if n not in want)
    wrong = sorted((n, where[n][1], tuple(want[n].shape)) for n in want
                   if n in where and tuple(where[n][1]) != tuple(want[n].shape))
    bad_dtype = sorted((n, where[n][2]) for n in want if n in where and where[n][2] not in
                       ("F32", "F64", "F16", "BF16", "I8", "I16", "I32", "I64", "U8"))
    if missing or unexpected or wrong or bad_dtype:
        raise WeightError(folder, missing, unexpected, wrong, bad_dtype)
    out: Dict[str, torch.Tensor] = {}
    by_file: Dict[str, List[str]] = {}
    for name in want:
        by_file.setdefault(where[name][0], []).append(name)
    for path, names in by_file.items():
        with safe_open(path, framework="pt", device="cpu") as fh:
            for name in names:
                t = fh.get_tensor(name)
                out[name] = t.to(device=device, dtype=stored_dtype(t.dtype))
    return out
