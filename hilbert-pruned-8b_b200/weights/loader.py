"""Binds a model's weight table to the tensors of a safetensors folder, by name.

The table (full tensor name -> expected shape and kind) comes from the model's parts.
Everything is checked before anything is copied, and all faults come in ONE error that
lists missing tensors, unexpected tensors and wrong shapes (the reference stops at the
first: ``weights: missing %s``, ``weights: %s has shape [a, b], expected [r, c]``,
cleanroom-transformer/src/model.c:226-244,272-281).  A tensor that no part asks for is not a
fault by itself: the reference never looks at what it does not bind (model.c:391-447), and
checkpoints carry extras (``mtp.*``, vision towers, ``rotary_emb.inv_freq``).  Such names are
still listed in the error when something else is wrong, where a misspelt name shows up as a
missing and an unexpected tensor side by side; ``strict=True`` makes them a fault of their own.

Dtype rule.  Serving precision (``bfloat16``): floating tensors stored in 16 bits are held
as bfloat16 (float16 is converted), a tensor stored in 32-bit stays 32-bit, integer tables
become int32.  ``float32``: every floating tensor is widened exactly to 32-bit
(model.c:259-270, ops_common.h:16-53).
"""
from __future__ import annotations

import fnmatch
from typing import Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

import torch

from ..parts.base import ParamSpec
from .safetensors_io import SafetensorsFolder

_TORCH_OF_TAG = {"F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "F64": torch.float64,
                 "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
                 "BOOL": torch.bool}

# tensors some exporters add that no part reads (the reference never asks for them)
DEFAULT_IGNORED = ("*.rotary_emb.inv_freq", "*.attention.bias", "*.attention.masked_bias")


class WeightError(ValueError):
    """All faults of a weight folder against a model's table, in one message."""

    def __init__(self, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 wrong_dtype: Sequence[Tuple[str, str]] = ()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = ["weights: the folder does not match the model"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, got, want in self.wrong_shape:
            lines.append(f"  {name} has shape {list(got)}, expected {list(want)}")
        for name, tag in self.wrong_dtype:
            lines.append(f"  {name} has dtype {tag}, which this tensor cannot be stored in")
        super().__init__("\n".join(lines))


def check_table(available: Mapping[str, Tuple[str, Tuple[int, ...]]], table: Mapping[str, ParamSpec],
                ignored: Iterable[str] = DEFAULT_IGNORED, strict: bool = False) -> List[str]:
    """Raises ``WeightError`` unless ``available`` (name -> (dtype tag, shape)) holds the
    table's tensors with the table's shapes; ``strict`` also refuses tensors the table does not
    name (but for the ``ignored`` patterns).  Returns the unexpected names."""
    missing: List[str] = []
    wrong: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]] = []
    wrong_dtype: List[Tuple[str, str]] = []
    for name, spec in table.items():
        if name not in available:
            if not spec.optional:
                missing.append(name)
            continue
        tag, shape = available[name]
        want = tuple(spec.shape)
        ok = tuple(shape) == want
        if spec.kind == "vector" and not ok:
            # a vector may be stored with extra unit dimensions (model.c:275-278 counts values)
            n = 1
            for s in shape:
                n *= s
            ok = n == want[0] and len(want) == 1
        if not ok:
            wrong.append((name, tuple(shape), want))
        floating = tag in ("F32", "F16", "BF16", "F64")
        if (spec.kind == "int_table") == floating:
            wrong_dtype.append((name, tag))
    patterns = list(ignored)
    unexpected = [n for n in available
                  if n not in table and not any(fnmatch.fnmatchcase(n, p) for p in patterns)]
    if missing or wrong or wrong_dtype or (strict and unexpected):
        raise WeightError(sorted(missing), sorted(unexpected), wrong, wrong_dtype)
    return sorted(unexpected)


def target_dtype(stored: torch.dtype, kind: str, precision: torch.dtype) -> torch.dtype:
    if kind == "int_table":
        return torch.int32
    if precision == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32          # a tensor stored in 32-bit stays so
    return torch.bfloat16


def load_tensors(model_dir: str, table: Mapping[str, ParamSpec], precision: torch.dtype,
                 device: torch.device, ignored: Iterable[str] = DEFAULT_IGNORED,
                 strict: bool = False) -> Dict[str, torch.Tensor]:
    """Checks the folder against ``table`` and returns the tensors on ``device``."""
    folder = SafetensorsFolder(model_dir)
    try:
        available = {n: (folder.entry(n).dtype, folder.entry(n).shape) for n in folder.names()}
        check_table(available, table, ignored, strict)
        out: Dict[str, torch.Tensor] = {}
        for name, spec in table.items():
            if name not in folder:
                continue
            src = folder.tensor(name)
            dst = target_dtype(src.dtype, spec.kind, precision)
            t = src.to(device=device, dtype=dst, copy=True)
            out[name] = t.reshape(spec.shape)
        return out
    finally:
        folder.close()


def choose_prefix(names: Iterable[str], prefixes: Sequence[str], probe: str) -> str:
    """The first of ``prefixes`` under which ``probe`` exists, else the last
    (cleanroom-transformer/src/model.c:394-395)."""
    have = set(names)
    for p in prefixes:
        if p + probe in have:
            return p
    return prefixes[-1]


def folder_names(model_dir: str) -> List[str]:
    folder = SafetensorsFolder(model_dir)
    try:
        return list(folder.names())
    finally:
        folder.close()
