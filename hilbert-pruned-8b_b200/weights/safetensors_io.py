"""Reader and writer for the safetensors container, by tensor name.

Format (cleanroom-transformer/src/safetensors.c:26-92): 8-byte little-endian header
length, a JSON header mapping each tensor name to ``dtype``, ``shape`` and
``data_offsets`` (relative to the end of the header), then the raw little-endian data.
A folder holds ``model.safetensors`` or the shards that ``model.safetensors.index.json``
lists under ``weight_map`` (safetensors.c:94-134).  Files are memory-mapped; tensors are
views into the mapping until the loader copies them to the device.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import torch


class SafetensorsError(ValueError):
    pass


# dtype tag -> (torch dtype, bytes per element)
_DTYPES = {
    "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_TAG_OF = {v[0]: k for k, v in _DTYPES.items()}


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    file: str
    begin: int  # absolute byte offsets in the file
    end: int


class SafetensorsFile:
    """One memory-mapped .safetensors file."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._fh = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"cannot open {path}: {e.strerror}") from None
        size = os.fstat(self._fh.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: bad header length")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen < 2 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: bad header length")
        try:
            header = json.loads(self._fh.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError):
            raise SafetensorsError(f"{path}: header is not valid JSON") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header is not an object")
        # private copy-on-write mapping: torch wants a writable buffer; the file is never changed
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_COPY)
        self.entries: Dict[str, TensorEntry] = {}
        base = 8 + hlen
        for name, info in header.items():
            if name == "__metadata__":
                continue
            try:
                tag, shape, (b, e) = info["dtype"], tuple(int(s) for s in info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: bad entry for {name}") from None
            if tag not in _DTYPES:
                continue  # dtypes the engine cannot hold are never asked for (safetensors.c:64-67)
            count = 1
            for s in shape:
                count *= s
            if b < 0 or e < b or base + e > size or e - b != count * _DTYPES[tag][1]:
                raise SafetensorsError(f"{path}: bad offsets for {name}")
            self.entries[name] = TensorEntry(name, tag, shape, path, base + b, base + e)

    def tensor(self, name: str) -> torch.Tensor:
        """A read-only CPU view of the tensor's bytes in its stored dtype."""
        e = self.entries[name]
        dtype, width = _DTYPES[e.dtype]
        count = (e.end - e.begin) // width
        if count == 0:
            return torch.empty(e.shape, dtype=dtype)
        t = torch.frombuffer(self._map, dtype=dtype, count=count, offset=e.begin)
        return t.view(e.shape)

    def close(self) -> None:
        # tensors handed out keep the mapping alive through the buffer protocol
        try:
            self._map.close()
        except (BufferError, ValueError):
            pass
        self._fh.close()


class SafetensorsFolder:
    """All tensors of a model folder, by name, across shards."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index = os.path.join(model_dir, "model.safetensors.index.json")
        files: List[str] = []
        if os.path.exists(index):
            with open(index, "r", encoding="utf-8") as f:
                try:
                    wm = json.load(f)["weight_map"]
                except (json.JSONDecodeError, KeyError, TypeError):
                    raise SafetensorsError(f"{index}: no weight_map") from None
            for shard in wm.values():
                if not isinstance(shard, str) or "/" in shard or shard.startswith("."):
                    raise SafetensorsError(f"{index}: bad shard name {shard!r}")
                if shard not in files:
                    files.append(shard)
        else:
            files.append("model.safetensors")
        self.files = [SafetensorsFile(os.path.join(model_dir, f)) for f in files]
        self._where: Dict[str, SafetensorsFile] = {}
        for fobj in self.files:
            for name in fobj.entries:
                self._where.setdefault(name, fobj)

    def names(self) -> Iterable[str]:
        return self._where.keys()

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def entry(self, name: str) -> TensorEntry:
        return self._where[name].entries[name]

    def tensor(self, name: str) -> torch.Tensor:
        return self._where[name].tensor(name)

    def close(self) -> None:
        for f in self.files:
            f.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    """Writes ``tensors`` (CPU or device; copied to the host one at a time) to ``path``."""
    header: Dict[str, dict] = {}
    offset = 0
    for name, t in tensors.items():
        if t.dtype not in _TAG_OF:
            raise SafetensorsError(f"cannot store dtype {t.dtype} of {name}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _TAG_OF[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for t in tensors.values():
            c = t.detach().contiguous().cpu()
            if c.numel():
                f.write(c.reshape(-1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)
