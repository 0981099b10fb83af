"""Python face of the CUDA kernel library: argument checks, dispatch, ctypes calls.

Every op runs a hand-written kernel on the current CUDA stream of ``torch``; torch itself
only owns the memory.  There is no CPU path and no library fallback: a missing library is
built on first use, and a failure to build or load it raises.

Dispatch rule for matrix products: the tensor-core kernel where its conditions hold
(bfloat16 operands, 16-byte aligned rows), else the general FP32-pipe kernel, which takes
every shape and dtype mix.  A kernel that cannot take a size refuses it with an error that
names the size; no op returns a wrong result for an odd size.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build
from .plan import decode_splits

_c_int, _c_ll, _c_float, _c_ptr = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p

_SIGNATURES = {
    "hb_device_info": [_c_int, ctypes.POINTER(_c_int), ctypes.POINTER(_c_int), ctypes.POINTER(_c_int)],
    "hb_timeline_set": [_c_ptr, _c_ptr, _c_int, _c_int],
    "hb_embed": [_c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    "hb_rmsnorm": [_c_ptr, _c_ptr, _c_float, _c_float, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_ptr],
    "hb_silu_mul": [_c_ptr, _c_int, _c_ll, _c_ptr, _c_int, _c_ll, _c_int, _c_int, _c_ptr],
    "hb_rope_table": [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr],
    "hb_rope_kv_append": [_c_ptr, _c_int, _c_ll, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_int,
                          _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    "hb_gemm_general": [_c_ptr, _c_int, _c_ll, _c_ptr, _c_int, _c_ll, _c_ptr, _c_int, _c_ll, _c_int, _c_int, _c_int,
                        _c_int, _c_ptr],
    "hb_gemm_tc": [_c_ptr, _c_ll, _c_ptr, _c_ll, _c_ll, _c_ptr, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                   _c_ptr, _c_ll, _c_ptr, _c_ll, _c_ptr, _c_int, _c_ptr],
    "hb_gemm_tc_fold": [_c_ptr, _c_ll, _c_ptr, _c_ll, _c_ll, _c_ptr, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                        _c_ptr, _c_ll, _c_ptr, _c_ll, _c_ptr, _c_int, _c_ptr, _c_ptr],
    "hb_gemm_tc2": [_c_ptr, _c_ll, _c_ptr, _c_ll, _c_ll, _c_ptr, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_int,
                    _c_ptr],
    "hb_attention_general": [_c_ptr, _c_int, _c_ll, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr,
                             _c_int, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_ptr, _c_ptr],
    "hb_attention_decode": [_c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ll, _c_int, _c_int,
                            _c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    "hb_attention_decode_combined": [_c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ll, _c_int,
                                     _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    "hb_attention_decode_fused": [_c_ptr, _c_ll, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr,
                                  _c_ll, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_int, _c_int,
                                  _c_ptr, _c_ptr],
    "hb_attention_prefill": [_c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ll, _c_int, _c_int,
                             _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_ptr, _c_ptr],
    "hb_attention_prefill_tc": [_c_ptr, _c_ll, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ll, _c_int,
                                _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_ptr, _c_ptr],
    "hb_random_normal": [_c_ptr, _c_int, _c_ll, ctypes.c_ulonglong, _c_float, _c_float, _c_ptr],
    "hb_argmax": [_c_ptr, _c_ll, _c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr],
    "hb_sample": [_c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr],
}

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
_lib = None


class KernelError(RuntimeError):
    pass


def load_library():
    """Loads (building first if needed) the kernel library; raises if that is impossible."""
    global _lib
    if _lib is None:
        path = build.library_path()
        lib = ctypes.CDLL(path)
        lib.hb_last_error.restype = ctypes.c_char_p
        lib.hb_last_error.argtypes = []
        for name, args in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = _c_int
        lib.hb_gemm_tc_token_tile.argtypes, lib.hb_gemm_tc_token_tile.restype = [_c_int], _c_int
        lib.hb_gemm_tc_scratch_floats.argtypes = [_c_int, _c_int, _c_int, _c_int, _c_int]
        lib.hb_gemm_tc_scratch_floats.restype = _c_ll
        lib.hb_gemm_tc_tiles.argtypes, lib.hb_gemm_tc_tiles.restype = [_c_int, _c_int, _c_int], _c_ll
        lib.hb_gemm_tc_resident_clusters.argtypes, lib.hb_gemm_tc_resident_clusters.restype = [_c_int, _c_int], _c_int
        lib.hb_gemm_tc2_wanted.argtypes, lib.hb_gemm_tc2_wanted.restype = [_c_int, _c_int, _c_int], _c_int
        lib.hb_gemm_tc2_resident_pairs.argtypes, lib.hb_gemm_tc2_resident_pairs.restype = [_c_int], _c_int
        for name in ("hb_attention_decode_supported", "hb_attention_prefill_supported", "hb_attention_prefill_tc_supported"):
            getattr(lib, name).argtypes, getattr(lib, name).restype = [_c_int, _c_int, _c_int], _c_int
        lib.hb_attention_decode_ctas_per_sm.argtypes, lib.hb_attention_decode_ctas_per_sm.restype = [_c_int], _c_int
        lib.hb_attention_decode_scratch_floats.argtypes = [_c_int, _c_int, _c_int, _c_int]
        lib.hb_attention_decode_scratch_floats.restype = _c_ll
        _lib = lib
    return _lib


def _code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not supported by the kernels") from None


def _rows(t: torch.Tensor, what: str) -> int:
    """Row stride of a 2-D tensor whose rows are contiguous."""
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelError(f"{what}: expected a 2-D tensor with contiguous rows, got shape {tuple(t.shape)} "
                          f"strides {t.stride()}")
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


class _NormFold(ctypes.Structure):
    """HbNormFold of csrc/api.h."""
    _fields_ = [("prep_w", ctypes.c_void_p), ("prep_offset", ctypes.c_float), ("prep_out", ctypes.c_void_p),
                ("prep_ld", ctypes.c_longlong), ("prep_sumsq", ctypes.c_void_p), ("scale_sumsq", ctypes.c_void_p),
                ("scale_parts", ctypes.c_int), ("scale_inv_size", ctypes.c_float), ("scale_eps", ctypes.c_float),
                ("sumsq_ld", ctypes.c_int)]


class PreparedNorm:
    """A norm whose input the product in front has prepared: the buffer it was asked to fill
    holds ``x * (offset + weight)`` without the per-token factor ``rsqrt(mean(x^2) + eps)``, and
    ``sumsq[token, :parts]`` add up to the token's sum of squares.  The product that reads the
    buffer multiplies its rows by the factor (``Ops.linear(..., scale=...)``)."""

    def __init__(self, sumsq: torch.Tensor, parts: int, size: int, eps: float):
        self.sumsq, self.parts, self.size, self.eps = sumsq, int(parts), int(size), float(eps)


class PackedWeight:
    """A bfloat16 weight matrix ``[rows, cols]`` stored for the tensor-core products: every
    128-row x 64-column tile is one contiguous 16 KB piece, and the tiles of a 128-row band
    follow one another along the columns (``data`` has the shape ``[bands, column blocks, 128,
    64]``, zero beyond ``rows`` and ``cols``).  A CTA that walks along the columns of a band
    then reads one sequential range of memory instead of 128 rows a whole matrix row apart.

    ``gate_up_bands``: the matrix is ``[gate; up]`` with halves of a multiple of 64 rows, and band
    ``b`` holds the gate rows ``64 b .. 64 b + 63`` followed by the up rows of the same features:
    what one tile of the fused SwiGLU product needs is then ONE piece (one tile load per K block
    instead of two, which a many-token product's K loop feels: 0.41 against 0.46 us per block)."""

    def __init__(self, data: torch.Tensor, rows: int, cols: int, gate_up_bands: bool = False):
        self.data, self.rows, self.cols, self.gate_up_bands = data, int(rows), int(cols), bool(gate_up_bands)

    @classmethod
    def pack(cls, w: torch.Tensor, gate_up_bands: bool = False) -> "PackedWeight":
        rows, cols = w.shape
        if gate_up_bands:
            half = rows // 2
            if rows % 2 or half % 64:
                raise KernelError(f"gate/up bands need halves of a multiple of 64 rows, not {rows} rows")
            banded = torch.stack([w[:half].view(half // 64, 64, cols), w[half:].view(half // 64, 64, cols)], dim=1)
            packed = cls.pack(banded.reshape(rows, cols))
            packed.gate_up_bands = True
            return packed
        bands, blocks = -(-rows // 128), -(-cols // 64)
        if rows % 128 or cols % 64:
            full = torch.zeros(bands * 128, blocks * 64, dtype=w.dtype, device=w.device)
            full[:rows, :cols] = w
            w = full
        return cls(w.view(bands, 128, blocks, 64).permute(0, 2, 1, 3).contiguous(), rows, cols)

    def unpacked(self) -> torch.Tensor:
        bands, blocks = self.data.shape[0], self.data.shape[1]
        w = self.data.permute(0, 2, 1, 3).reshape(bands * 128, blocks * 64)[: self.rows, : self.cols]
        if self.gate_up_bands:
            w = w.reshape(self.rows // 128, 2, 64, self.cols).transpose(0, 1).reshape(self.rows, self.cols)
        return w.contiguous()

    def first_rows(self, n: int) -> "PackedWeight":
        """The matrix of the first ``n`` rows (shares the storage)."""
        if not 0 < n <= self.rows or self.gate_up_bands:
            raise KernelError(f"first_rows: {n} of {self.rows} rows" + (" of a [gate; up] matrix in bands" if self.gate_up_bands else ""))
        return PackedWeight(self.data, n, self.cols)

    @property
    def shape(self):
        return (self.rows, self.cols)

    @property
    def dtype(self):
        return self.data.dtype

    @property
    def device(self):
        return self.data.device

    def numel(self) -> int:
        return self.rows * self.cols

    def element_size(self) -> int:
        return self.data.element_size()

    def data_ptr(self) -> int:
        return self.data.data_ptr()


class Ops:
    """The kernels bound to one device."""

    def __init__(self, device):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise KernelError("the kernels run on a CUDA device only")
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device is available; the library has no CPU path")
        self.lib = load_library()
        self.call_log = None  # a list: the name of every library call is appended (diagnostics)
        major, minor, sms = _c_int(), _c_int(), _c_int()
        idx = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self._call("hb_device_info", idx, ctypes.byref(major), ctypes.byref(minor), ctypes.byref(sms))
        self.sm = (major.value, minor.value)
        self.sm_count = sms.value
        if major.value != 10:
            raise KernelError(f"the kernels are built for sm_100a; device {idx} is sm_{major.value}{minor.value}")
        self.launches = 0  # kernels launched through this object (a claim bench.py reports)
        self.use_tensor_cores = True   # tests switch this off to compare the two matrix-product kernels
        self.use_pair_gemm = True      # many-token products on CTA pairs (cta_group::2)
        # few-token steps: a norm between two products is folded into them (HILBERT_B200_FOLD_NORMS=0: norm kernels)
        self.fold_norms = os.environ.get("HILBERT_B200_FOLD_NORMS", "1") != "0"
        self._sumsq = None             # [FOLD_MAX_TOKENS, slots]: the partial sums of squares of a folded norm
        # weights as contiguous tiles (PackedWeight); HILBERT_B200_PACK=0 keeps them row-major
        self.use_packed_weights = os.environ.get("HILBERT_B200_PACK", "1") != "0"
        # device status words (csrc/common.cuh): a kernel that meets a fault notes the first one of
        # its kind and carries on with a safe value; the host reads the words where it waits anyway
        # (check_errors, or copied back beside a step's sampled tokens) and raises
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.error_flag = self.status[:1]      # word 0: a bounded wait of a tensor-core kernel ran out
        # split-K scratch: float32 partial tiles and one counter per output tile (kept zero)
        self._splitk_partials = torch.empty(8 << 20, dtype=torch.float32, device=self.device)
        self._splitk_counters = torch.zeros(1 << 16, dtype=torch.int32, device=self.device)
        # split-K decode attention scratch: partial outputs with their maxima and sums
        self._decode_scratch = torch.empty(4 << 20, dtype=torch.float32, device=self.device)
        self._decode_counters = torch.zeros(1 << 16, dtype=torch.int32, device=self.device)
        # greedy pick: (maximum, index) of each range of a row, and a counter per row (kept zero)
        self._argmax_scratch = torch.empty(2 * 1024 * self.ARGMAX_MAX_PARTS, dtype=torch.int32, device=self.device)
        self._argmax_counters = torch.zeros(1024, dtype=torch.int32, device=self.device)
        self._retired = []              # outgrown scratch, kept alive for graphs that captured it
        self._splits_cache = {}
        self.use_tcgen05_attention = True   # head size 128 prefill on tcgen05 (else the mma.sync kernel)
        self.use_fast_attention = True  # tests switch this off to compare with the general kernel
        # Decode attention that rotates the new queries and key and appends to the cache itself
        # (no rotation kernel in front; the new key and value go into the owning split's copy of
        # their page in shared memory).  Inside a replayed graph at batch 8 / 8192 tokens it takes
        # 43.2 us where rotation + attention take 3.4 + 41.0 us; alternating runs on one GPU, a step
        # of 8 layers: 1310 against 1312 us, at batch 1 1046 against 1047 us, 1B sizes 613 against
        # 616 us.  One launch less, the time of the hand-over between kernels stays.  Whether a
        # model's attention uses it is the part's choice (the mixer's `fuse_decode`, its position
        # encoding's `fusable`); this switch only takes the kernel away (tests compare both ways).
        self.fuse_decode_attention = True
        # Split-K decode attention whose last split combines the splits, instead of a second
        # kernel.  Off: at batch 8 / 8192 tokens a step of 8 layers takes 1319 us against 1313 us, at
        # batch 1 1079 against 1052 us (the last split's two round trips are longer than a kernel
        # that is already resident); with the rotation inside as well, 50.3 us per layer against
        # 43.2 + 3.5 us.  A single split always writes the result itself.
        self.combine_in_attention = False

    # ------------------------------------------------------------------ plumbing
    def _call(self, name: str, *args) -> None:
        rc = getattr(self.lib, name)(*args)
        if rc != 0:
            raise KernelError(self.lib.hb_last_error().decode("utf-8", "replace"))
        if self.call_log is not None:
            self.call_log.append(name)

    # ------------------------------------------------------------------ timeline
    def timeline_begin(self, capacity: int = 1 << 16, events: bool = False) -> None:
        """Switches the kernels' time marks on (library built with HILBERT_B200_TIMELINE=1 only):
        from now on every kernel notes when its first block reached its dependency wait and
        when that wait returned.  ``events`` also records the events inside the kernels that have
        some (the few-token matrix product); they cost those kernels a few microseconds."""
        self._tl_marks = torch.zeros(capacity, 2, dtype=torch.int64, device=self.device)
        self._tl_count = torch.zeros(1, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)
        self._call("hb_timeline_set", self._tl_marks.data_ptr(), self._tl_count.data_ptr(), capacity,
                   1 if events else 0)

    def timeline_end(self):
        """Switches the marks off; returns the marks ordered by their second field.  A kernel's
        mark is (resident_ns, predecessors_done_ns) of its first block; an event inside a kernel
        (the matrix product has some) is (code * 1000 + block, time_ns) with a first field
        below 10**9."""
        torch.cuda.synchronize(self.device)
        self._call("hb_timeline_set", None, None, 0, 0)
        n = min(int(self._tl_count.item()), self._tl_marks.shape[0])
        marks = self._tl_marks[:n].tolist()
        self._tl_marks = self._tl_count = None
        return sorted(((a, b) for a, b in marks), key=lambda m: m[1])

    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def _dev(self, *tensors) -> None:
        for t in tensors:
            if t is not None and t.device != self.device:
                raise KernelError(f"tensor on {t.device}, kernels bound to {self.device}")

    # ------------------------------------------------------------------ elementwise
    def embed(self, tokens, table, out) -> None:
        """``out[t] = table[tokens[t]]`` widened to 32-bit; ``table`` row-major or a PackedWeight."""
        packed = isinstance(table, PackedWeight)
        self._dev(tokens, table.data if packed else table, out)
        if tokens.dtype != torch.int32 or out.dtype != torch.float32 or not out.is_contiguous() \
                or not (packed or table.is_contiguous()):
            raise KernelError("embed: tokens int32, contiguous table, contiguous float32 output expected")
        T, H = out.shape
        if table.shape[1] != H or tokens.numel() != T:
            raise KernelError("embed: shapes do not agree")
        self._call("hb_embed", tokens.data_ptr(), table.data_ptr(), _code(table), out.data_ptr(), T, H,
                   table.shape[0], 1 if packed else 0, self.status.data_ptr(), self._stream())
        self.launches += 1

    def rmsnorm(self, x, weight, eps: float, offset: float, out, rows=None) -> None:
        self._dev(x, weight, out, rows)
        if x.dtype != torch.float32 or weight.dtype != torch.float32 or not x.is_contiguous() \
                or not out.is_contiguous() or not weight.is_contiguous():
            raise KernelError("rmsnorm: contiguous float32 input and weight, contiguous output expected")
        H = x.shape[1]
        n = out.shape[0]
        if out.shape[1] != H or weight.numel() != H:
            raise KernelError("rmsnorm: shapes do not agree")
        if rows is None:
            if n != x.shape[0]:
                raise KernelError("rmsnorm: output rows differ from input rows")
            rp = None
        else:
            if rows.dtype != torch.int32 or rows.numel() != n:
                raise KernelError("rmsnorm: rows must be int32, one per output row")
            rp = rows.data_ptr()
        self._call("hb_rmsnorm", x.data_ptr(), weight.data_ptr(), float(eps), float(offset), out.data_ptr(), _code(out),
                   rp, n, H, self._stream())
        self.launches += 1

    def silu_mul(self, gate_up, out) -> None:
        self._dev(gate_up, out)
        inter = out.shape[1]
        if gate_up.shape[1] != 2 * inter or gate_up.shape[0] != out.shape[0]:
            raise KernelError("silu_mul: input must be [rows, 2 * inter]")
        self._call("hb_silu_mul", gate_up.data_ptr(), _code(gate_up), _rows(gate_up, "silu_mul input"), out.data_ptr(),
                   _code(out), _rows(out, "silu_mul output"), out.shape[0], inter, self._stream())
        self.launches += 1

    def rope_table(self, positions, inv_freq, out) -> None:
        self._dev(positions, inv_freq, out)
        T, half = out.shape[0], out.shape[1]
        if positions.dtype != torch.int32 or positions.numel() != T or inv_freq.dtype != torch.float32 \
                or inv_freq.numel() != half or out.dtype != torch.float32 or not out.is_contiguous() \
                or out.shape[2] != 2:
            raise KernelError("rope_table: shapes or dtypes do not agree")
        self._call("hb_rope_table", positions.data_ptr(), inv_freq.data_ptr(), out.data_ptr(), T, half, self._stream())
        self.launches += 1

    def rope_kv_append(self, qkv, table, rot: int, heads: int, kv_heads: int, head_dim: int, cache, step,
                       append: bool) -> None:
        self._dev(qkv, table, cache.k, cache.v)
        T = qkv.shape[0]
        need = (heads + (2 * kv_heads if append else 0)) * head_dim
        if qkv.shape[1] < need:
            raise KernelError("rope_kv_append: qkv rows are too short")
        pt = step.page_tables[cache.group]
        if rot and (table is None or table.shape[0] != T or table.shape[1] != rot // 2):
            raise KernelError("rope_kv_append: rotary table does not match the tokens")
        if cache.k.dtype != cache.v.dtype or not cache.k.is_contiguous() or not cache.v.is_contiguous():
            raise KernelError("rope_kv_append: cache layers must be contiguous and of one dtype")
        if tuple(cache.k.shape[1:]) != (kv_heads, 64, head_dim):
            raise KernelError(f"rope_kv_append: cache layer shape {tuple(cache.k.shape)} does not match "
                              f"{kv_heads} kv heads of size {head_dim}")
        self._call("hb_rope_kv_append", qkv.data_ptr(), _code(qkv), _rows(qkv, "qkv"),
                   table.data_ptr() if rot else None, rot, heads, kv_heads, head_dim, cache.k.data_ptr(),
                   cache.v.data_ptr(), _code(cache.k), pt.data_ptr(), pt.shape[1], step.tok_seq.data_ptr(),
                   step.positions.data_ptr(), T, 1 if append else 0, cache.k.shape[0], self.status.data_ptr(),
                   self._stream())
        self.launches += 1

    STATUS_WORDS = 4

    @staticmethod
    def status_message(words) -> Optional[str]:
        """What the status words say, or None if all are zero."""
        w = [int(x) for x in words]
        if not any(w):
            return None
        parts = []
        if w[0]:
            parts.append(f"a tensor-core kernel gave up a bounded wait (code {w[0]}); its results are invalid")
        if w[1]:
            parts.append(f"non-finite logits at row {w[1] - 1} of a step (the reference fails such a row too)")
        if w[2]:
            parts.append(f"a page number outside the cache, or a missing page, for sequence {w[2] - 1} of a step: "
                         "the cache's bookkeeping is at fault")
        if w[3]:
            parts.append(f"a token id outside the vocabulary at row {w[3] - 1} of a step")
        return "; ".join(parts)

    def raise_on_status(self, words) -> None:
        """Raises ``KernelError`` for non-zero status words that were read already (a host copy),
        after clearing the device's words and the split-K counters a kernel that gave up may have
        left non-zero."""
        msg = self.status_message(words)
        if msg is not None:
            self.reset_status()
            raise KernelError(msg)

    def reset_status(self) -> None:
        self.status.zero_()
        self._splitk_counters.zero_()
        self._decode_counters.zero_()
        self._argmax_counters.zero_()

    def check_errors(self) -> None:
        """Reads the device status words (this synchronises) and raises if a kernel noted a fault."""
        self.raise_on_status(self.status.tolist())

    # ------------------------------------------------------------------ matrix products
    def pack_weight(self, w: torch.Tensor, swiglu: bool = False):
        """``w`` as a PackedWeight when the tensor-core products can read it that way (bfloat16
        on this device, rows of a multiple of 8 elements; a [gate; up] matrix needs halves of a
        multiple of 64 rows), else ``w`` itself."""
        if (not self.use_packed_weights or not isinstance(w, torch.Tensor) or w.dtype != torch.bfloat16 or w.dim() != 2
                or w.device != self.device or w.shape[1] % 8 or (swiglu and (w.shape[0] // 2) % 64)):
            return w
        return PackedWeight.pack(w, gate_up_bands=swiglu)

    def _tensor_core_operands(self, a, w) -> bool:
        if not (self.use_tensor_cores and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and _rows(a, "linear input") % 8 == 0):
            return False
        return isinstance(w, PackedWeight) or _rows(w, "linear weight") % 8 == 0

    SCHEDULES = {None: 0, "auto": 0, "tiles": 1, "stream_k": 2, "cut_first": 3}

    def _gemm_tc(self, a, w, out, mode: int, N: int, up_row0: int = 0, schedule=None, fold=None) -> None:
        M, K = a.shape
        packed = 1 if isinstance(w, PackedWeight) else 0
        ldw = 64 if packed else _rows(w, "linear weight")
        if fold is None and (schedule == "pairs" or (schedule is None and self.use_pair_gemm and self.lib.hb_gemm_tc2_wanted(M, N, K)
                                                     and not (mode == 3 and N % 8))):
            # many tokens: CTA pairs (cta_group::2) on 256 x 256 tiles
            self._call("hb_gemm_tc2", a.data_ptr(), _rows(a, "linear input"), w.data_ptr(), ldw, w.shape[0], out.data_ptr(),
                       _rows(out, "linear output"), M, N, K, mode, up_row0, self.error_flag.data_ptr(), packed, self._stream())
            self.launches += 1
            return
        sched = self.SCHEDULES[schedule]
        need = self.lib.hb_gemm_tc_scratch_floats(M, N, K, mode, sched)
        tiles = self.lib.hb_gemm_tc_tiles(M, N, mode)
        if need > self._splitk_partials.numel():
            self._retired.append(self._splitk_partials)     # a captured graph may still write there
            self._splitk_partials = torch.empty(need, dtype=torch.float32, device=self.device)
        if tiles > self._splitk_counters.numel():
            self._retired.append(self._splitk_counters)
            self._splitk_counters = torch.zeros(tiles, dtype=torch.int32, device=self.device)
        args = (a.data_ptr(), _rows(a, "linear input"), w.data_ptr(), ldw,
                w.shape[0], out.data_ptr(), _rows(out, "linear output"), M, N, K, mode, up_row0, sched,
                self._splitk_partials.data_ptr(), self._splitk_partials.numel(), self._splitk_counters.data_ptr(),
                self._splitk_counters.numel(), self.error_flag.data_ptr(), packed)
        if fold is None:
            self._call("hb_gemm_tc", *args, self._stream())
        else:
            self._call("hb_gemm_tc_fold", *args, ctypes.byref(fold), self._stream())    # the library copies the values
        self.launches += 1

    # ------------------------------------------------------------------ a norm folded into the products around it
    FOLD_MAX_TOKENS = 32           # TC_SCALE_ROWS of csrc/tcgen05.cuh: beyond, norm kernels are as fast or faster

    def can_fold_norm(self, tokens: int, size: int, dtype: torch.dtype) -> bool:
        """Whether a step of ``tokens`` tokens may fold a norm over vectors of ``size`` into the
        products around it: few tokens (the few-token tensor-core kernel), bfloat16 activations."""
        return bool(self.fold_norms and self.use_tensor_cores and dtype == torch.bfloat16 and 0 < tokens <= self.FOLD_MAX_TOKENS
                    and size % 8 == 0)

    def _sumsq_buffer(self, size: int) -> torch.Tensor:
        ld = (-(-size // 32) + 3) // 4 * 4
        if self._sumsq is None or self._sumsq.shape[1] < ld:
            if self._sumsq is not None:
                self._retired.append(self._sumsq)            # a captured graph may still write there
            self._sumsq = torch.zeros(self.FOLD_MAX_TOKENS, ld, dtype=torch.float32, device=self.device)
        return self._sumsq

    def _prepare_fold(self, out, prepare) -> Optional[_NormFold]:
        """The producer's half of HbNormFold, or None when this product cannot prepare the norm."""
        weight, offset, eps, h_out = prepare
        M, N = out.shape
        if not (self.can_fold_norm(M, N, h_out.dtype) and out.dtype == torch.float32 and out.data_ptr() % 16 == 0
                and _rows(out, "linear output") % 4 == 0 and weight.dtype == torch.float32 and weight.numel() == N
                and weight.data_ptr() % 16 == 0 and tuple(h_out.shape) == (M, N) and h_out.data_ptr() % 8 == 0
                and _rows(h_out, "norm output") % 4 == 0):
            return None
        sumsq = self._sumsq_buffer(N)
        fold = _NormFold()
        fold.prep_w, fold.prep_offset, fold.prep_out = weight.data_ptr(), float(offset), h_out.data_ptr()
        fold.prep_ld, fold.prep_sumsq, fold.sumsq_ld = _rows(h_out, "norm output"), sumsq.data_ptr(), sumsq.shape[1]
        return fold

    def _scale_fold(self, scale: PreparedNorm, tokens: int) -> _NormFold:
        if tokens > self.FOLD_MAX_TOKENS:
            raise KernelError(f"a prepared norm serves up to {self.FOLD_MAX_TOKENS} tokens, not {tokens}")
        fold = _NormFold()
        fold.scale_sumsq, fold.scale_parts, fold.sumsq_ld = scale.sumsq.data_ptr(), scale.parts, scale.sumsq.shape[1]
        fold.scale_inv_size, fold.scale_eps = 1.0 / scale.size, scale.eps
        return fold

    def linear(self, a, w, out, accumulate: bool = False, schedule=None, prepare=None, scale: Optional[PreparedNorm] = None):
        """``out[M,N] (+)= a[M,K] @ w[N,K]^T`` with float32 accumulation.  ``schedule`` forces
        the tensor-core kernel's work split ("tiles" or "stream_k"; default: by shape).

        A norm folded into the products around it (few tokens, bfloat16): with ``accumulate`` and
        ``prepare = (norm weight, offset, eps, buffer)`` the product also fills ``buffer`` with
        ``out * (offset + weight)`` and returns a ``PreparedNorm`` (None when it cannot: the
        caller then runs the norm).  ``scale``: ``a`` is such a buffer; the rows of the result are
        multiplied by the norm's per-token factor."""
        self._dev(a, w, out)
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K or tuple(out.shape) != (M, N):
            raise KernelError(f"linear: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} do not agree")
        if isinstance(w, PackedWeight) and w.gate_up_bands:
            raise KernelError("linear: a [gate; up] matrix stored in bands is an operand of linear_swiglu only")
        if self._tensor_core_operands(a, w) and (out.dtype == torch.float32 or not accumulate):
            mode = 2 if accumulate else (1 if out.dtype == torch.float32 else 0)
            fold = None
            if prepare is not None and accumulate and schedule != "pairs":
                fold = self._prepare_fold(out, prepare)
            if scale is not None:
                if accumulate:
                    raise KernelError("linear: the product that adds to the residual does not scale its rows")
                fold = self._scale_fold(scale, M)
            self._gemm_tc(a, w, out, mode, N, 0, schedule, fold=fold)
            if fold is not None and scale is None:
                return PreparedNorm(self._sumsq, -(-N // 32), N, prepare[2])
            return None
        if scale is not None:
            raise KernelError("linear: operands that the tensor-core product refuses cannot take a prepared norm")
        if isinstance(w, PackedWeight):
            w = w.unpacked()           # not a product path: only operands the tensor-core kernels refuse get here
        self._call("hb_gemm_general", a.data_ptr(), _code(a), _rows(a, "linear input"), w.data_ptr(), _code(w),
                   _rows(w, "linear weight"), out.data_ptr(), _code(out), _rows(out, "linear output"), M, N, K,
                   1 if accumulate else 0, self._stream())
        self.launches += 1

    def linear_swiglu(self, h, w_gate_up, act, workspace, cap: int, schedule=None, scale: Optional[PreparedNorm] = None) -> None:
        """``act = silu(h Wg^T) * (h Wu^T)`` with ``w_gate_up = [Wg; Wu]``; ``scale`` as in ``linear``."""
        T = h.shape[0]
        inter = act.shape[1]
        if w_gate_up.shape[0] != 2 * inter or act.shape[0] != T:
            raise KernelError("linear_swiglu: weight must be [2 * inter, hidden]")
        if (self._tensor_core_operands(h, w_gate_up) and act.dtype == torch.bfloat16 and act.data_ptr() % 16 == 0
                and _rows(act, "swiglu output") % 8 == 0):
            bands = isinstance(w_gate_up, PackedWeight) and w_gate_up.gate_up_bands
            self._gemm_tc(h, w_gate_up, act, 3, inter, up_row0=-1 if bands else inter, schedule=schedule,
                          fold=self._scale_fold(scale, T) if scale is not None else None)
            return
        if scale is not None:
            raise KernelError("linear_swiglu: operands that the tensor-core product refuses cannot take a prepared norm")
        if isinstance(w_gate_up, PackedWeight):
            w_gate_up = w_gate_up.unpacked()
        gu = workspace.buffer("swiglu.gate_up", (cap, 2 * inter), torch.float32 if act.dtype == torch.float32
                              else torch.bfloat16)[:T]
        self.linear(h, w_gate_up, gu)
        self.silu_mul(gu, act)

    # ------------------------------------------------------------------ attention
    def decode_splits_for(self, batch: int, kv_heads: int, max_pages: int, head_dim: int = 128) -> int:
        """Key splits of decode attention (``plan.decode_splits``) for this device: the CTAs it
        holds at once are the kernel's CTAs per SM (two at head size 128) times its SMs."""
        key = (batch, kv_heads, max_pages, head_dim)
        hit = self._splits_cache.get(key)
        if hit is None:
            slots = self.sm_count * max(1, self.lib.hb_attention_decode_ctas_per_sm(head_dim) or 2)
            hit = self._splits_cache[key] = decode_splits(batch, kv_heads, max_pages, slots)
        return hit

    def can_fuse_decode_attention(self, qkv, heads: int, kv_heads: int, head_dim: int, cache, step, out) -> bool:
        """Whether ``attention_decode_fused`` takes this step: one token per sequence,
        bfloat16 everywhere, a head size and group the tensor-core kernel is built for."""
        return bool(self.fuse_decode_attention and self.use_fast_attention and step.is_decode
                    and qkv.dtype == torch.bfloat16
                    and cache.k.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
                    and cache.k.is_contiguous() and cache.v.is_contiguous()
                    and step.num_tokens * kv_heads <= self._decode_counters.numel()
                    and self.lib.hb_attention_decode_supported(heads, kv_heads, head_dim))

    def attention_decode_fused(self, qkv, table, rot: int, heads: int, kv_heads: int, head_dim: int, cache, step, out,
                               scale: float, window: Optional[int], append: bool, splits: Optional[int] = None) -> None:
        """Rotation of the new tokens' queries and keys, cache append and split-K attention in
        one launch (decode steps only); the combination of the splits is a second kernel, or
        with ``combine_in_attention`` the work of the last split to finish.  ``qkv`` holds
        the projections before rotation and is not written."""
        self._dev(qkv, table, cache.k, cache.v, out)
        T = qkv.shape[0]
        pt = step.page_tables[cache.group]
        if out.shape[0] != T or out.shape[1] != heads * head_dim:
            raise KernelError("attention: output shape does not match")
        if rot and (table is None or table.shape[0] != T or table.shape[1] != rot // 2):
            raise KernelError("attention: rotary table does not match the tokens")
        if tuple(cache.k.shape[1:]) != (kv_heads, 64, head_dim):
            raise KernelError("attention: cache layer shape does not match the heads")
        max_pages = (step.max_len + 63) // 64
        n_splits = splits if splits is not None else self.decode_splits_for(T, kv_heads, max_pages, head_dim)
        n_splits = max(1, min(n_splits, max_pages))
        need = self.lib.hb_attention_decode_scratch_floats(T, heads, head_dim, n_splits)
        if need > self._decode_scratch.numel():
            self._retired.append(self._decode_scratch)
            self._decode_scratch = torch.empty(need, dtype=torch.float32, device=self.device)
        self._call("hb_attention_decode_fused", qkv.data_ptr(), _rows(qkv, "attention projections"),
                   table.data_ptr() if rot else None, rot, cache.k.data_ptr(), cache.v.data_ptr(), pt.data_ptr(),
                   pt.shape[1], step.positions.data_ptr(), self._decode_scratch.data_ptr(),
                   self._decode_counters.data_ptr() if self.combine_in_attention else None,
                   out.data_ptr(), _rows(out, "attention output"), T, heads, kv_heads,
                   head_dim, float(scale), int(window) if window else 0, n_splits, max_pages, cache.k.shape[0],
                   1 if append else 0, self.status.data_ptr(), self._stream())
        self.launches += 1 if (n_splits == 1 or self.combine_in_attention) else 2

    def attention(self, qkv, heads: int, kv_heads: int, head_dim: int, cache, step, out, scale: float,
                  window: Optional[int], splits: Optional[int] = None) -> None:
        """Causal attention of the step's tokens over the cache; queries are the first
        ``heads * head_dim`` columns of ``qkv``.  bfloat16 with head size 64 or 128 runs the
        tensor-core kernels (split-K for one token per sequence, flash-style otherwise);
        everything else runs the general kernel."""
        self._dev(qkv, cache.k, cache.v, out)
        T = qkv.shape[0]
        pt = step.page_tables[cache.group]
        if out.shape[0] != T or out.shape[1] != heads * head_dim:
            raise KernelError("attention: output shape does not match")
        win = int(window) if window else 0
        fast = (self.use_fast_attention and qkv.dtype == torch.bfloat16 and cache.k.dtype == torch.bfloat16
                and out.dtype == torch.bfloat16 and cache.k.is_contiguous() and cache.v.is_contiguous())
        if fast and step.is_decode and self.lib.hb_attention_decode_supported(heads, kv_heads, head_dim):
            max_pages = (step.max_len + 63) // 64
            n_splits = splits if splits is not None else self.decode_splits_for(T, kv_heads, max_pages, head_dim)
            n_splits = max(1, min(n_splits, max_pages))
            need = self.lib.hb_attention_decode_scratch_floats(T, heads, head_dim, n_splits)
            if need > self._decode_scratch.numel():
                self._retired.append(self._decode_scratch)
                self._decode_scratch = torch.empty(need, dtype=torch.float32, device=self.device)
            if ((n_splits == 1 or self.combine_in_attention) and n_splits <= 16
                    and T * kv_heads <= self._decode_counters.numel()):
                # one split writes the result itself; with more, the last split of a (sequence, kv
                # head) to finish can combine them (a switch: measured slower than the second kernel)
                self._call("hb_attention_decode_combined", qkv.data_ptr(), _rows(qkv, "attention queries"), cache.k.data_ptr(),
                           cache.v.data_ptr(), pt.data_ptr(), pt.shape[1], step.positions.data_ptr(),
                           self._decode_scratch.data_ptr(), self._decode_counters.data_ptr(), out.data_ptr(),
                           _rows(out, "attention output"), T, heads, kv_heads, head_dim, float(scale), win, n_splits, max_pages,
                           cache.k.shape[0], self.status.data_ptr(), self._stream())
                self.launches += 1
                return
            self._call("hb_attention_decode", qkv.data_ptr(), _rows(qkv, "attention queries"), cache.k.data_ptr(),
                       cache.v.data_ptr(), pt.data_ptr(), pt.shape[1], step.positions.data_ptr(),
                       self._decode_scratch.data_ptr(), out.data_ptr(), _rows(out, "attention output"), T, heads, kv_heads,
                       head_dim, float(scale), win, n_splits, max_pages, cache.k.shape[0], self.status.data_ptr(),
                       self._stream())
            self.launches += 2
            return
        if (fast and self.use_tcgen05_attention and self.lib.hb_attention_prefill_tc_supported(heads, kv_heads, head_dim)
                and qkv.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0 and _rows(qkv, "attention queries") % 8 == 0
                and _rows(out, "attention output") % 8 == 0
                and sum((n + 127) // 128 for n in step.host_new) <= 65535):
            q_blocks = sum((n + 127) // 128 for n in step.host_new)
            self._call("hb_attention_prefill_tc", qkv.data_ptr(), _rows(qkv, "attention queries"), T, cache.k.data_ptr(),
                       cache.v.data_ptr(), pt.data_ptr(), pt.shape[1], step.seq_start.data_ptr(), step.seq_pos0.data_ptr(),
                       out.data_ptr(), _rows(out, "attention output"), step.num_seqs, q_blocks, heads, kv_heads, head_dim,
                       float(scale), win, cache.k.shape[0], self.error_flag.data_ptr(), self._stream())
            self.launches += 1
            return
        if (fast and self.lib.hb_attention_prefill_supported(heads, kv_heads, head_dim)
                and sum((n + 63) // 64 for n in step.host_new) <= 65535):
            q_blocks = sum((n + 63) // 64 for n in step.host_new)
            self._call("hb_attention_prefill", qkv.data_ptr(), _rows(qkv, "attention queries"), cache.k.data_ptr(),
                       cache.v.data_ptr(), pt.data_ptr(), pt.shape[1], step.seq_start.data_ptr(), step.seq_pos0.data_ptr(),
                       out.data_ptr(), _rows(out, "attention output"), step.num_seqs, q_blocks, heads, kv_heads, head_dim,
                       float(scale), win, cache.k.shape[0], self.status.data_ptr(), self._stream())
            self.launches += 1
            return
        self._call("hb_attention_general", qkv.data_ptr(), _code(qkv), _rows(qkv, "attention queries"),
                   cache.k.data_ptr(), cache.v.data_ptr(), _code(cache.k), pt.data_ptr(), pt.shape[1],
                   step.tok_seq.data_ptr(), step.positions.data_ptr(), out.data_ptr(), _code(out),
                   _rows(out, "attention output"), T, heads, kv_heads, head_dim, float(scale), win, cache.k.shape[0],
                   self.status.data_ptr(), self._stream())
        self.launches += 1

    # ------------------------------------------------------------------ random weights
    def random_normal(self, out, base: int, std: float, mean: float = 0.0) -> None:
        """``out.flat[i] = mean + std * N(0, 1)``, element ``i`` of the counter-based stream
        ``base`` (``weights.random_init.stream_base``): the values the CPU draws, bit for bit."""
        self._dev(out)
        if not out.is_contiguous():
            raise KernelError("random_normal: contiguous output expected")
        self._call("hb_random_normal", out.data_ptr(), _code(out), out.numel(), int(base) & ((1 << 64) - 1), float(std),
                   float(mean), self._stream())
        self.launches += 1

    # ------------------------------------------------------------------ sampling
    ARGMAX_MAX_PARTS = 16

    def argmax(self, logits, out) -> None:
        """``out[r]`` = index of the largest value of row r (the lowest index on ties).  A row is cut
        over several blocks when there are fewer rows than the device has room for."""
        self._dev(logits, out)
        n = logits.shape[0]
        if logits.dtype != torch.float32 or out.dtype != torch.int32 or out.numel() != n:
            raise KernelError("argmax: float32 logits and one int32 per row expected")
        parts = max(1, min(self.ARGMAX_MAX_PARTS, (2 * self.sm_count) // max(n, 1), logits.shape[1] // 4096))
        if n > self._argmax_counters.numel():
            self._retired += [self._argmax_counters, self._argmax_scratch]      # a captured graph may still use them
            self._argmax_counters = torch.zeros(n, dtype=torch.int32, device=self.device)
            self._argmax_scratch = torch.empty(2 * n * self.ARGMAX_MAX_PARTS, dtype=torch.int32, device=self.device)
        self._call("hb_argmax", logits.data_ptr(), _rows(logits, "logits"), out.data_ptr(), n, logits.shape[1], parts,
                   self._argmax_scratch.data_ptr(), self._argmax_counters.data_ptr(), self.status.data_ptr(), self._stream())
        self.launches += 1

    def sample(self, logits, temperature, seeds, request_ids, steps, out) -> None:
        self._dev(logits, temperature, seeds, request_ids, steps, out)
        n = logits.shape[0]
        if logits.dtype != torch.float32 or out.dtype != torch.int32 or temperature.dtype != torch.float32 \
                or any(t.dtype != torch.int64 for t in (seeds, request_ids, steps)) \
                or any(t.numel() != n for t in (temperature, seeds, request_ids, steps, out)):
            raise KernelError("sample: float32 logits/temperature, int64 seeds/requests/steps, int32 output, "
                              "one of each per row expected")
        self._call("hb_sample", logits.data_ptr(), _rows(logits, "logits"), temperature.data_ptr(), seeds.data_ptr(),
                   request_ids.data_ptr(), steps.data_ptr(), out.data_ptr(), n, logits.shape[1], self.status.data_ptr(),
                   self._stream())
        self.launches += 1
