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
        self.capturing = False      # set while a CUDA graph is being captured
        self._pinned = set()        # buffers whose addresses a captured graph holds: they must not move

    def buffer(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        numel = 1
        for s in shape:
            numel *= int(s)
        key = f"{name}|{dtype}"
        flat = self._buffers.get(key)
        if self.capturing:
            if flat is None or flat.numel() < numel:
                raise RuntimeError(f"workspace: buffer {name} would be allocated inside a graph capture")
            self._pinned.add(key)
        if flat is None or flat.numel() < numel:
            if key in self._pinned:
                raise RuntimeError(f"workspace: buffer {name} would move while a captured graph uses it")
            flat = torch.empty(max(numel, 1), dtype=dtype, device=self.device)
            self._buffers[key] = flat
        return flat[:numel].view(shape)

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._buffers.values())
