"""Random-weights mode: tensors for a model's weight table from a seed, and a writer that
turns a configuration and a seed into a model folder (config.json + model.safetensors).

The reference has no such mode in the engine; its tests draw random checkpoints in PyTorch
(cleanroom-transformer/tools/parity.py:58-69).  Matrices are N(0, std); norm vectors are 1
or 1 + N(0, norm_std).  Tensors are drawn in table order from one generator, so a seed
names one model for a given table and device type.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Mapping, Optional

import torch

from ..parts.base import ParamSpec
from .safetensors_io import write_safetensors


def random_tensors(table: Mapping[str, ParamSpec], seed: int, device: torch.device,
                   std: float = 0.02, norm_std: float = 0.0, dtype: torch.dtype = torch.bfloat16,
                   fan_in_scale: Optional[float] = None) -> Dict[str, torch.Tensor]:
    """``fan_in_scale`` s: matrices get std ``s / sqrt(columns)`` instead of ``std``
    (weights large enough that every layer moves the logits)."""
    device = torch.device(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    out: Dict[str, torch.Tensor] = {}
    for name, spec in table.items():
        if spec.optional:
            continue
        shape = tuple(spec.shape)
        if spec.kind == "int_table":
            out[name] = torch.zeros(shape, dtype=torch.int32, device=device)
        elif spec.init == "ones":
            t = torch.ones(shape, dtype=torch.float32, device=device)
            if norm_std:
                t += torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * norm_std
            out[name] = t.to(dtype)
        elif spec.init == "zeros":
            out[name] = torch.zeros(shape, dtype=dtype, device=device)
        else:
            s = std if fan_in_scale is None or len(shape) < 2 else fan_in_scale / float(shape[-1]) ** 0.5
            t = torch.empty(shape, dtype=torch.float32, device=device)
            # drawn in slabs so that a vocabulary-sized matrix needs no second full copy
            rows = max(1, (1 << 26) // max(1, t[0].numel())) if t.dim() > 1 else t.shape[0]
            for r0 in range(0, shape[0], rows):
                part = t[r0:r0 + rows]
                part.copy_(torch.randn(part.shape, generator=gen, device=device, dtype=torch.float32) * s)
            out[name] = t.to(dtype)
    return out


def write_random_model(model_dir: str, config, seed: int, std: float = 0.02, norm_std: float = 0.0,
                       dtype: torch.dtype = torch.bfloat16, fan_in_scale: Optional[float] = None) -> str:
    """Writes ``model_dir/config.json`` and ``model_dir/model.safetensors`` for ``config``."""
    from ..engine.model import weight_table  # the table is the model's, not the writer's
    os.makedirs(model_dir, exist_ok=True)
    spec = config.model_spec()
    table = weight_table(spec, prefix=spec.weight_prefixes[-1])
    tensors = random_tensors(table, seed, torch.device("cpu"), std, norm_std, dtype, fan_in_scale)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=1)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors)
    return model_dir
