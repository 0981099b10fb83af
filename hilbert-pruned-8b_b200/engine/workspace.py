"""Scratch buffers that live as long as the engine.

A part asks for a buffer by name with the largest shape it will ever need (the step-token
capacity) and slices it; the same name gives the same memory at every step, so a captured
CUDA graph stays valid and the hot path allocates nothing.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch


class Workspace:
    def __init__(self, device):
        self.device = device
        self._buffers: Dict[str, torch.Tensor] = {}
        self.frozen = False  # set while CUDA graphs that captured these addresses are alive

    def buffer(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        numel = 1
        for s in shape:
            numel *= int(s)
        key = f"{name}|{dtype}"
        flat = self._buffers.get(key)
        if flat is None or flat.numel() < numel:
            if self.frozen and flat is not None:
                raise RuntimeError(f"workspace: buffer {name} would move while a captured graph uses it")
            flat = torch.empty(max(numel, 1), dtype=dtype, device=self.device)
            self._buffers[key] = flat
        return flat[:numel].view(shape)

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._buffers.values())
