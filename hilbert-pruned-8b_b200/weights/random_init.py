"""Random-weights mode: tensors for a model's weight table from a seed, and a writer that
turns a configuration and a seed into a model folder (config.json + model.safetensors).

The reference has no such mode in the engine; its tests draw random checkpoints in PyTorch
and share the files (cleanroom-transformer/tools/parity.py:58-69,115-142).  Here every
element is a FUNCTION of ``(seed, tensor name, element index)``: a counter-based generator,
no stream.  The same seed therefore names the same model, bit for bit, whether it is drawn
on the CPU (this file, NumPy) or on the GPU (``csrc/random_init.cu``), in whatever order and
for whatever subset of the table; a model drawn on the device can be handed to anything
that reads a folder written on the CPU with the same seed.

The draw, in 32-bit arithmetic whose every operation rounds the same way on both sides
(add, multiply, divide, square root: no library logarithm or cosine, no fused multiply-add):

* ``key`` = FNV-1a (64 bit) of the tensor's full name; ``base = mix(seed * G + key * M1 + C)``;
  element ``i`` hashes to ``z = mix(base + (i + 1) * G)`` (the SplitMix64 sequence from ``base``).
* the top 32 bits of ``z`` give a probability ``p = (k + 0.5) * 2**-33`` in (0, 0.5], bit 0 the sign.
* ``x = sign * Phi^-1(p)`` by Acklam's rational approximation of the normal quantile (relative
  error 1.2e-9 in exact arithmetic, about 1e-6 in 32-bit); its tail needs ``log p``, computed from
  the exponent and the series of ``atanh`` for the mantissa.
* value = ``mean + std * x`` in 32-bit, rounded to nearest-even if the tensor is bfloat16.

Matrices are N(0, std) (or std ``fan_in_scale / sqrt(columns)``); norm vectors are 1 or
1 + N(0, norm_std); integer tables are zero.
"""
from __future__ import annotations

import concurrent.futures
import json
import os
from typing import Dict, Mapping, Optional

import numpy as np
import torch

from ..parts.base import ParamSpec
from .safetensors_io import write_safetensors

_M64 = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15
_MUL1 = 0xBF58476D1CE4E5B9
_MUL2 = 0x94D049BB133111EB
_ADD = 0x2545F4914F6CDD1D

# Acklam's coefficients, rounded once to 32-bit (csrc/random_init.cu carries the same values
# as hexadecimal literals)
_F = np.float32
_A = [_F(x) for x in (-3.969683028665376e+01, 2.209460984245205e+02, -2.759285104469687e+02,
                      1.383577518672690e+02, -3.066479806614716e+01, 2.506628277459239e+00)]
_B = [_F(x) for x in (-5.447609879822406e+01, 1.615858368580409e+02, -1.556989798598866e+02,
                      6.680131188771972e+01, -1.328068155288572e+01)]
_C = [_F(x) for x in (-7.784894002430293e-03, -3.223964580411365e-01, -2.400758277161838e+00,
                      -2.549732539343734e+00, 4.374664141464968e+00, 2.938163982698783e+00)]
_D = [_F(x) for x in (7.784695709041462e-03, 3.224671290700398e-01, 2.445134137142996e+00,
                      3.754408661907416e+00)]
_P_LOW = _F(0.02425)
_LN2 = _F(0.6931471805599453)
_SQRT_HALF = _F(0.7071067811865476)
_THIRD, _FIFTH, _SEVENTH, _NINTH = _F(1.0 / 3.0), _F(1.0 / 5.0), _F(1.0 / 7.0), _F(1.0 / 9.0)
_ONE, _TWO, _HALF = _F(1.0), _F(2.0), _F(0.5)
_CHUNK = 1 << 20


def _mix64_int(z: int) -> int:
    z = ((z ^ (z >> 30)) * _MUL1) & _M64
    z = ((z ^ (z >> 27)) * _MUL2) & _M64
    return z ^ (z >> 31)


def name_key(name: str) -> int:
    """FNV-1a, 64 bit, of the tensor's name."""
    h = 0xCBF29CE484222325
    for byte in name.encode("utf-8"):
        h = ((h ^ byte) * 0x100000001B3) & _M64
    return h


def stream_base(seed: int, name: str) -> int:
    """The 64-bit state from which a tensor's elements are hashed."""
    return _mix64_int(((seed & _M64) * _GOLDEN + name_key(name) * _MUL1 + _ADD) & _M64)


def _log32(p: np.ndarray) -> np.ndarray:
    """Natural logarithm of positive normal 32-bit numbers from exactly rounded operations:
    ``p = m * 2**e`` with m in [sqrt(1/2), sqrt(2)), ``log m = 2 atanh((m - 1) / (m + 1))``."""
    bits = p.view(np.uint32)
    e = (bits >> np.uint32(23)).astype(np.int32) - np.int32(126)
    m = ((bits & np.uint32(0x007FFFFF)) | np.uint32(0x3F000000)).view(np.float32)      # [0.5, 1)
    small = m < _SQRT_HALF
    m = np.where(small, m * _TWO, m)
    e = np.where(small, e - np.int32(1), e)
    t = (m - _ONE) / (m + _ONE)
    t2 = t * t
    s = t2 * _NINTH + _SEVENTH
    s = s * t2 + _FIFTH
    s = s * t2 + _THIRD
    s = s * t2 + _ONE
    return (_TWO * t) * s + e.astype(np.float32) * _LN2


def standard_normals(base: int, start: int, count: int) -> np.ndarray:
    """Elements ``start .. start + count`` of the stream ``base`` as 32-bit standard normals."""
    with np.errstate(over="ignore"):
        i = np.arange(start + 1, start + count + 1, dtype=np.uint64)
        z = np.uint64(base) + i * np.uint64(_GOLDEN)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(_MUL1)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(_MUL2)
        z = z ^ (z >> np.uint64(31))
    negative = (z & np.uint64(1)).astype(bool)
    k = (z >> np.uint64(32)).astype(np.uint32)
    p = (k.astype(np.float32) + _HALF) * _F(2.0 ** -33)
    # centre: p >= p_low
    q = p - _HALF
    r = q * q
    num = _A[0]
    for c in _A[1:]:
        num = num * r + c
    den = _B[0]
    for c in _B[1:]:
        den = den * r + c
    x = (num * q) / (den * r + _ONE)
    tail = p < _P_LOW
    if tail.any():
        pt = p[tail]
        qt = np.sqrt(_F(-2.0) * _log32(pt))
        num = _C[0]
        for c in _C[1:]:
            num = num * qt + c
        den = _D[0]
        for c in _D[1:]:
            den = den * qt + c
        x[tail] = num / (den * qt + _ONE)
    # x is the quantile of p <= 1/2, so it is <= 0: the sign bit mirrors it
    return np.where(negative, x, -x).astype(np.float32, copy=False)


def normal_tensor_cpu(shape, seed: int, name: str, std: float, mean: float, dtype: torch.dtype) -> torch.Tensor:
    """``mean + std * N(0, 1)`` of the stream ``(seed, name)`` on the CPU, in ``dtype``."""
    n = 1
    for s in shape:
        n *= int(s)
    base = stream_base(seed, name)
    flat = np.empty(n, dtype=np.float32)
    std32, mean32 = _F(std), _F(mean)

    def fill(lo: int) -> None:
        hi = min(n, lo + _CHUNK)
        flat[lo:hi] = standard_normals(base, lo, hi - lo) * std32 + mean32

    starts = range(0, n, _CHUNK)
    if n > 4 * _CHUNK:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 1)) as pool:
            list(pool.map(fill, starts))
    else:
        for lo in starts:
            fill(lo)
    return torch.from_numpy(flat).view(tuple(shape)).to(dtype)


def random_tensors(table: Mapping[str, ParamSpec], seed: int, device: torch.device,
                   std: float = 0.02, norm_std: float = 0.0, dtype: torch.dtype = torch.bfloat16,
                   fan_in_scale: Optional[float] = None, ops=None) -> Dict[str, torch.Tensor]:
    """The table's tensors for ``seed``, on ``device`` (a CUDA device draws them with the
    kernel library: ``ops``, or one made for the purpose; the values are the CPU's, bit for bit).
    ``fan_in_scale`` s: matrices get std ``s / sqrt(columns)`` instead of ``std`` (weights large
    enough that every layer moves the logits)."""
    device = torch.device(device)
    if device.type == "cuda" and ops is None:
        from ..kernels.ops import Ops
        ops = Ops(device)
    out: Dict[str, torch.Tensor] = {}

    def draw(name, shape, s, mean, dt):
        if device.type == "cuda":
            t = torch.empty(shape, dtype=dt, device=device)
            ops.random_normal(t, stream_base(seed, name), s, mean)
            return t
        return normal_tensor_cpu(shape, seed, name, s, mean, dt)

    for name, spec in table.items():
        if spec.optional:
            continue
        shape = tuple(spec.shape)
        if spec.kind == "int_table":
            out[name] = torch.zeros(shape, dtype=torch.int32, device=device)
        elif spec.init == "ones":
            out[name] = draw(name, shape, norm_std, 1.0, dtype) if norm_std else torch.ones(shape, dtype=dtype, device=device)
        elif spec.init == "zeros":
            out[name] = torch.zeros(shape, dtype=dtype, device=device)
        else:
            s = std if fan_in_scale is None or len(shape) < 2 else fan_in_scale / float(shape[-1]) ** 0.5
            out[name] = draw(name, shape, s, 0.0, dtype)
    return out


def write_random_model(model_dir: str, config, seed: int, std: float = 0.02, norm_std: float = 0.0,
                       dtype: torch.dtype = torch.bfloat16, fan_in_scale: Optional[float] = None,
                       device="cpu") -> str:
    """Writes ``model_dir/config.json`` and ``model_dir/model.safetensors`` for ``config``.
    ``device``: where the values are drawn (a CUDA device is much faster for a large model; the
    file is the same, bit for bit)."""
    from ..engine.model import weight_table  # the table is the model's, not the writer's
    os.makedirs(model_dir, exist_ok=True)
    spec = config.model_spec()
    table = weight_table(spec, prefix=spec.weight_prefixes[-1])
    tensors = random_tensors(table, seed, torch.device(device), std, norm_std, dtype, fan_in_scale)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=1)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors)
    return model_dir
