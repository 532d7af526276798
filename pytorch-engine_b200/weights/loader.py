"""Weights from safetensors, by tensor name.

What a model needs is read off its plan: every part declares its weights (shape and role), the
plan maps them to checkpoint tensor names.  The file set is ``model.safetensors`` or the shards
named by ``model.safetensors.index.json``.  One check compares the two sides and reports, in a
single error, every missing tensor, every unexpected tensor and every wrong shape.

Storage types: 16-bit floats are kept as bfloat16 (float16 as float32 when the run is a float32 one:
float16 has three more mantissa bits than bfloat16, and the float32 path is there to show what rounding
hides), a tensor stored in 32-bit floats stays float32, 64-bit floats become float32, integer tables
become int32.  A tensor's role decides what it may be stored as: a matrix, an embedding or a norm weight
stored as integers is refused, and so is an integer table stored as floats (the reference refuses tensor
types it does not know, pygguf_engine/gguf_parser.py:250-256).

Tensors the plan does not name are errors, with two exceptions that the plan itself declares:
``plan.duplicates`` (a name that may be in the file if it holds the same values as another tensor: a tied
model whose file also stores ``lm_head.weight``) and ``plan.ignored`` (name patterns of buffers that carry
no weights, such as stored rotary frequencies).

(The reference reads GGUF by name, pygguf_engine/gguf_parser.py:236-267, floats via
pygguf_engine/quant_kernels.py:1097-1116; a missing tensor is a bare KeyError there.)
"""
from __future__ import annotations

import fnmatch
import json
import os
from typing import Dict, List, Optional, Tuple

import torch

from ..parts.registry import lookup
from ..parts.spec import ModelPlan, WeightDecl


class WeightError(ValueError):
    """The checkpoint does not match the model; ``missing``, ``unexpected`` and ``wrong_shape`` list how."""

    def __init__(self, folder: str, missing, unexpected, wrong_shape, bad_dtype=(), conflicting=()) -> None:
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.bad_dtype = list(bad_dtype)
        self.conflicting = list(conflicting)
        lines = [f"checkpoint in {folder!r} does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: file has {list(got)}, model wants {list(want)}" for n, got, want in self.wrong_shape))
        if self.bad_dtype:
            lines.append(f"  unusable dtypes ({len(self.bad_dtype)}): " + "; ".join(
                f"{n}: stored as {dt}, a {role} must be stored as {want}" for n, dt, role, want in self.bad_dtype))
        if self.conflicting:
            lines.append(f"  duplicates that differ ({len(self.conflicting)}): " + "; ".join(
                f"{n} must equal {other}" for n, other in self.conflicting))
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
_FLOAT_TAGS = ("F32", "F64", "F16", "BF16")
_INT_TAGS = ("I8", "I16", "I32", "I64", "U8")


def stored_dtype(dtype: torch.dtype, run_dtype: Optional[torch.dtype] = None) -> torch.dtype:
    """The dtype a stored tensor is kept in after loading (see the module text)."""
    if dtype == torch.float16 and run_dtype == torch.float32:
        return torch.float32
    if dtype in _FLOAT_KEEP:
        return _FLOAT_KEEP[dtype]
    if dtype in _INT_TYPES:
        return torch.int32
    raise TypeError(str(dtype))


def usable_tags(role: str) -> Tuple[str, ...]:
    """The safetensors dtype tags a tensor of ``role`` may be stored as."""
    return _INT_TAGS if role == "table_int" else _FLOAT_TAGS


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


def load_weights(folder: str, plan: ModelPlan, device="cpu", dtype: Optional[torch.dtype] = None) -> Dict[str, torch.Tensor]:
    """{checkpoint name: tensor on ``device``} for every tensor the plan needs, after the check.
    ``dtype``: the run dtype (it only decides what float16 tensors are kept as)."""
    from safetensors import safe_open

    want = expected_tensors(plan)
    duplicates = dict(getattr(plan, "duplicates", None) or {})
    ignored = tuple(getattr(plan, "ignored", None) or ())
    files = _files_of(folder)
    where: Dict[str, Tuple[str, Tuple[int, ...], str]] = {}
    for path in files:
        if not os.path.isfile(path):
            raise FileNotFoundError(f"model.safetensors.index.json names {os.path.basename(path)!r}, which is not in {folder!r}")
        with safe_open(path, framework="pt", device="cpu") as fh:
            for name in fh.keys():
                sl = fh.get_slice(name)
                where[name] = (path, tuple(sl.get_shape()), sl.get_dtype())
    missing = sorted(n for n in want if n not in where)
    extra = [n for n in where if n not in want]
    check_equal = sorted(n for n in extra if n in duplicates and duplicates[n] in want)
    unexpected = sorted(n for n in extra if n not in check_equal and not any(fnmatch.fnmatchcase(n, pat) for pat in ignored))
    wrong = sorted((n, where[n][1], tuple(want[n].shape)) for n in want
                   if n in where and tuple(where[n][1]) != tuple(want[n].shape))
    bad_dtype = sorted((n, where[n][2], want[n].role, " / ".join(usable_tags(want[n].role))) for n in want
                       if n in where and where[n][2] not in usable_tags(want[n].role))
    conflicting = []
    for n in check_equal:
        other = duplicates[n]
        if other not in where:
            continue
        if where[n][1] != where[other][1]:
            conflicting.append((n, other))
            continue
        with safe_open(where[n][0], framework="pt", device="cpu") as fa, safe_open(where[other][0], framework="pt", device="cpu") as fb:
            if not torch.equal(fa.get_tensor(n), fb.get_tensor(other)):
                conflicting.append((n, other))
    if missing or unexpected or wrong or bad_dtype or conflicting:
        raise WeightError(folder, missing, unexpected, wrong, bad_dtype, conflicting)
    out: Dict[str, torch.Tensor] = {}
    by_file: Dict[str, List[str]] = {}
    for name in want:
        by_file.setdefault(where[name][0], []).append(name)
    for path, names in by_file.items():
        with safe_open(path, framework="pt", device="cpu") as fh:
            for name in names:
                t = fh.get_tensor(name)
                out[name] = t.to(device=device, dtype=stored_dtype(t.dtype, dtype))
    return out
