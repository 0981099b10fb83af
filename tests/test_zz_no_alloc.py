"""The decode-attention entry point that allocates nothing (csrc/noalloc.h), called through
its exported C symbol as a plug-in without an allocator would call it: inputs and output
come from the caller, the split-K scratch is the library's built-in device array.  Its
output must equal that of the ordinary entry point (which gets scratch from the caller) on
two calls in a row with different inputs, whether this file runs alone or last."""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _lib():
    from hilbert_pruned_8b_b200.kernels import build
    lib = ctypes.CDLL(build.library_path())
    P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    lib.hb_last_error.restype = ctypes.c_char_p
    lib.hb_attention_decode.argtypes = [P, L, P, P, P, I, P, P, P, L, I, I, I, I, F, I, I, I, I, P, P]
    lib.hb_attention_decode_noalloc.argtypes = [P, L, P, P, P, I, P, P, L, I, I, I, I, F, I, I, I, I, P]
    lib.hb_attention_decode_scratch_floats.argtypes = [I, I, I, I]
    lib.hb_attention_decode_scratch_floats.restype = L
    return lib


def _case(seed, batch, nh, nkv, hd, lengths, n_pages):
    g = torch.Generator(device=DEV).manual_seed(seed)
    k = torch.randn(n_pages, nkv, 64, hd, generator=g, device=DEV).to(torch.bfloat16)
    v = torch.randn(n_pages, nkv, 64, hd, generator=g, device=DEV).to(torch.bfloat16)
    q = torch.randn(batch, nh * hd, generator=g, device=DEV).to(torch.bfloat16)
    width = max((n + 63) // 64 for n in lengths)
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    table = torch.full((batch, width), -1, dtype=torch.int32)
    for b, n in enumerate(lengths):
        for p in range((n + 63) // 64):
            table[b, p] = perm.pop()
    positions = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)
    return q, k, v, table.to(DEV), positions, width


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    nh, nkv, hd, splits = 8, 2, 128, 3
    for seed, lengths in ((1, [130, 1, 64, 300]), (2, [65, 257, 19, 128])):
        batch = len(lengths)
        q, k, v, table, positions, width = _case(seed, batch, nh, nkv, hd, lengths, 24)
        scale = 1.0 / math.sqrt(hd)
        scratch = torch.empty(lib.hb_attention_decode_scratch_floats(batch, nh, hd, splits), device=DEV)
        want = torch.zeros(batch, nh * hd, device=DEV, dtype=torch.bfloat16)
        rc = lib.hb_attention_decode(q.data_ptr(), nh * hd, k.data_ptr(), v.data_ptr(), table.data_ptr(), width,
                                     positions.data_ptr(), scratch.data_ptr(), want.data_ptr(), nh * hd, batch, nh, nkv, hd,
                                     scale, 0, splits, width, 24, None, stream)
        assert rc == 0, lib.hb_last_error()
        got = torch.full_like(want, 7.0)
        rc = lib.hb_attention_decode_noalloc(q.data_ptr(), nh * hd, k.data_ptr(), v.data_ptr(), table.data_ptr(), width,
                                             positions.data_ptr(), got.data_ptr(), nh * hd, batch, nh, nkv, hd, scale, 0,
                                             splits, width, 24, stream)
        assert rc == 0, lib.hb_last_error()
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        err = (got.double() - want.double()).abs().max().item() / want.double().abs().max().item()
        assert err < 2 ** -7, f"call with seed {seed}: relative difference {err:.3e}"
        # and against a plain statement of attention, so that both are not wrong together
        for b, n in enumerate(lengths):
            pages = table[b, :(n + 63) // 64].long()
            kk = k[pages].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[:, :n].double()
            vv = v[pages].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[:, :n].double()
            for j in range(nh):
                sc = (kk[j // (nh // nkv)] @ q[b, j * hd:(j + 1) * hd].double()) * scale
                ref = torch.softmax(sc, 0) @ vv[j // (nh // nkv)]
                assert (got[b, j * hd:(j + 1) * hd].double() - ref).abs().max() < 2 ** -7 * ref.abs().max() + 1e-3


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    lib = _lib()
    dummy = torch.zeros(16, device=DEV)
    rc = lib.hb_attention_decode_noalloc(dummy.data_ptr(), 4096, dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), 64,
                                         dummy.data_ptr(), dummy.data_ptr(), 4096, 4096, 32, 8, 128, 0.1, 0, 8, 64, 1, None)
    assert rc != 0
    msg = lib.hb_last_error().decode()
    assert "scratch floats" in msg and "built-in area" in msg


def test_no_alloc_entry_point_reads_nothing_beyond_the_page_table():
    """A position that lies beyond what the page table covers (a caller's mistake): the kernel
    reads the pages the table has and nothing past its end; more pages per sequence than the
    table is wide are refused before anything runs."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    nh, nkv, hd, splits = 8, 2, 128, 2
    q, k, v, table, positions, width = _case(3, 2, nh, nkv, hd, [100, 40], 24)
    table = table[:, :2].contiguous()                       # two pages per sequence, then the next row starts
    positions = torch.tensor([500, 39], dtype=torch.int32, device=DEV)      # 500 is far beyond 2 * 64
    got = torch.full((2, nh * hd), 7.0, device=DEV, dtype=torch.bfloat16)
    rc = lib.hb_attention_decode_noalloc(q.data_ptr(), nh * hd, k.data_ptr(), v.data_ptr(), table.data_ptr(), 2,
                                         positions.data_ptr(), got.data_ptr(), nh * hd, 2, nh, nkv, hd, 0.1, 0, splits, 2, 24,
                                         stream)
    assert rc == 0, lib.hb_last_error()
    torch.cuda.synchronize()
    assert torch.isfinite(got.float()).all()
    rc = lib.hb_attention_decode_noalloc(q.data_ptr(), nh * hd, k.data_ptr(), v.data_ptr(), table.data_ptr(), 2,
                                         positions.data_ptr(), got.data_ptr(), nh * hd, 2, nh, nkv, hd, 0.1, 0, splits, 8, 24,
                                         stream)
    assert rc != 0 and "page table of width 2" in lib.hb_last_error().decode()
