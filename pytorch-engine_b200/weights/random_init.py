"""Random-weights mode: a model folder (config.json + model.safetensors) from a configuration and a seed.

Matrices and embeddings are drawn from N(0, 0.02), norm weights from 1 + N(0, 0.02) so that no
norm weight is trivially one.  Every tensor has a generator stream of its own, keyed by the seed
and the tensor's name, so the values do not depend on the order in which tensors are made.  Values
are rounded to bfloat16 (the type they are stored in).  Tensors made directly on a CUDA device
(``random_weights(..., device="cuda")``, used for shapes too large to write to disk quickly) come
from the device's generator and differ from the host's values for the same seed.
"""
from __future__ import annotations

import hashlib
import os
from typing import Dict

import torch

from ..config.base import ModelConfig
from ..config.registry import architecture
from ..parts.spec import ModelPlan
from .loader import expected_tensors

WEIGHT_STD = 0.02


def _stream_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_weights(plan: ModelPlan, seed: int, device="cpu", norm_dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    device = torch.device(device)
    out: Dict[str, torch.Tensor] = {}
    for name, decl in expected_tensors(plan).items():
        gen = torch.Generator(device=device)
        gen.manual_seed(_stream_seed(seed, name))
        if decl.role == "table_int":
            out[name] = torch.zeros(decl.shape, dtype=torch.int32, device=device)
            continue
        if device.type == "cuda" and len(decl.shape) == 2 and decl.shape[0] * decl.shape[1] > (1 << 28):
            # very large tables: fill in row blocks to bound the float32 temporary
            t = torch.empty(decl.shape, dtype=torch.bfloat16, device=device)
            rows = max(1, (1 << 27) // decl.shape[1])
            for r0 in range(0, decl.shape[0], rows):
                r1 = min(decl.shape[0], r0 + rows)
                t[r0:r1] = (torch.randn((r1 - r0, decl.shape[1]), generator=gen, device=device) * WEIGHT_STD).to(torch.bfloat16)
            out[name] = t
            continue
        x = torch.randn(decl.shape, generator=gen, device=device, dtype=torch.float32) * WEIGHT_STD
        if decl.role == "norm":
            out[name] = (1.0 + x).to(torch.bfloat16).to(norm_dtype)
        else:
            out[name] = x.to(torch.bfloat16)
    return out


def write_random_model(folder: str, config: ModelConfig, seed: int, norm_dtype: torch.dtype = torch.bfloat16) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` with weights from ``seed``."""
    from safetensors.torch import save_file

    arch = architecture(config.architecture)
    plan = arch.plan(config)
    os.makedirs(folder, exist_ok=True)
    config.save(folder)
    tensors = random_weights(plan, seed, "cpu", norm_dtype)
    save_file({k: v.contiguous() for k, v in tensors.items()}, os.path.join(folder, "model.safetensors"),
              metadata={"format": "pt", "seed": str(seed)})
    return folder
