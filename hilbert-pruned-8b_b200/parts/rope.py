"""Rotary position encoding with optional llama3 frequency scaling.

``inv_freq[i] = 1 / theta^(2i/rot)`` in 32-bit, then the llama3 rule per frequency: long
wavelengths divided by ``factor``, short ones kept, the band between interpolated
(cleanroom-transformer/src/model.c:450-469).  At position p the pair ``(i, i + rot/2)`` of
each head is rotated by ``inv_freq[i] * float(p)`` (cpu_backend.c:87-98).  The table of
frequencies is made once on the host; cosines and sines of a step's positions are made
once per step on the device and shared by every layer that uses the same parameters.
"""
from __future__ import annotations

import numpy as np
import torch

from .base import POSITION_ENCODINGS, PositionEncoding


def rotary_inv_freq(rotary_dim: int, theta: float, llama3=None) -> np.ndarray:
    f32 = np.float32
    k = np.arange(rotary_dim // 2, dtype=np.float32)
    expo = (f32(2.0) * k) / f32(rotary_dim)
    freq = (f32(1.0) / np.power(f32(theta), expo, dtype=np.float32)).astype(np.float32)
    if llama3 is not None:
        factor = f32(llama3["factor"])
        low = f32(llama3["low_freq_factor"])
        high = f32(llama3["high_freq_factor"])
        orig = f32(llama3["original_max_position_embeddings"])
        pi = f32(3.14159265358979323846)
        out = np.empty_like(freq)
        for i, f in enumerate(freq):
            wavelen = f32(2.0) * pi / f
            low_wavelen = orig / low
            high_wavelen = orig / high
            scaled = f / factor if wavelen > low_wavelen else f
            if not (wavelen < high_wavelen) and not (wavelen > low_wavelen):
                smooth = (orig / wavelen - low) / (high - low)
                scaled = (f32(1.0) - smooth) * scaled / factor + smooth * scaled
            out[i] = f32(scaled)
        freq = out
    return freq.astype(np.float32)


@POSITION_ENCODINGS.register("rotary")
class RotaryEmbedding(PositionEncoding):
    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.head_dim = int(spec.params["head_dim"])
        self.rotary_dim = int(spec.params["rotary_dim"])
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary: rotary_dim {self.rotary_dim} does not fit head_dim {self.head_dim}")
        self.inv_freq_host = rotary_inv_freq(self.rotary_dim, float(spec.params["theta"]), spec.get("llama3"))
        self._inv_freq = None
        self._key = "rope:" + repr(spec)

    @property
    def inv_freq(self) -> torch.Tensor:
        if self._inv_freq is None:
            self._inv_freq = torch.from_numpy(self.inv_freq_host.copy()).to(self.ctx.device)
        return self._inv_freq

    def prepare(self, step) -> None:
        if self._key in step.shared:
            return
        half = self.rotary_dim // 2
        table = self.ctx.workspace.buffer(self._key, (self.ctx.max_step_tokens, half, 2), torch.float32)
        table = table[: step.num_tokens]
        self.ctx.ops.rope_table(step.positions, self.inv_freq, table)
        step.shared[self._key] = table

    def rotation_table(self, step):
        """``([tokens, rot/2, 2] cosines and sines of this step's positions, rot)``."""
        self.prepare(step)
        return step.shared[self._key], self.rotary_dim
