"""Each kernel alone against a plain torch statement of the same operation, at sizes other
than the engine's tiny models (widths and vocabularies that are no power of two, head sizes
in steps of 16, odd head and group counts)."""
import math
import types

import pytest
import torch

from conftest import require_gpu

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    require_gpu()
    from hilbert_pruned_8b_b200.kernels.ops import Ops
    return Ops(torch.device(DEV))


def _bf(x):
    return x.to(torch.bfloat16)


def _rel(got, ref):
    return ((got.double() - ref.double()).abs().max() / ref.double().abs().max().clamp(min=1e-6)).item()


# ------------------------------------------------------------------------------- elementwise
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(ops, dtype):
    torch.manual_seed(0)
    table = torch.randn(301, 72, device=DEV).to(dtype)
    toks = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 72, device=DEV)
    ops.embed(toks, table, out)
    assert torch.equal(out, table[toks.long()].float())
    if dtype == torch.bfloat16:
        # the same rows from the table stored as tiles (what a tied head keeps): one copy serves both
        for rows, cols in ((301, 72), (1000, 200), (128, 64)):
            t2 = torch.randn(rows, cols, device=DEV).to(dtype)
            ids = torch.tensor([0, rows - 1, 127 % rows, 128 % rows, 5], dtype=torch.int32, device=DEV)
            o2 = torch.empty(5, cols, device=DEV)
            ops.embed(ids, ops.pack_weight(t2), o2)
            assert torch.equal(o2, t2[ids.long()].float())


@pytest.mark.parametrize("hidden,eps,offset", [(72, 1e-5, 0.0), (1000, 1e-6, 1.0), (4096, 1e-5, 0.0)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm(ops, hidden, eps, offset, out_dtype):
    torch.manual_seed(1)
    x = torch.randn(7, hidden, device=DEV) * 3
    w = torch.randn(hidden, device=DEV)
    ref = x.double() / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + eps) * (offset + w.double())
    out = torch.empty(7, hidden, device=DEV, dtype=out_dtype)
    ops.rmsnorm(x, w, eps, offset, out)
    tol = 2e-6 if out_dtype == torch.float32 else 2 ** -8
    assert _rel(out, ref) < tol
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    sub = torch.empty(3, hidden, device=DEV, dtype=out_dtype)
    ops.rmsnorm(x, w, eps, offset, sub, rows)
    assert torch.equal(sub, out[rows.long()])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_mul(ops, dtype):
    torch.manual_seed(2)
    gu = (torch.randn(9, 2 * 176, device=DEV) * 4).to(dtype)
    out = torch.empty(9, 176, device=DEV, dtype=dtype)
    ops.silu_mul(gu, out)
    g, u = gu[:, :176].double(), gu[:, 176:].double()
    ref = g / (1 + torch.exp(-g)) * u
    assert _rel(out, ref) < (1e-6 if dtype == torch.float32 else 2 ** -8)


def test_rope_table(ops):
    pos = torch.tensor([0, 1, 63, 64, 5000, 131071], dtype=torch.int32, device=DEV)
    inv = (1.0 / (500000.0 ** (torch.arange(0, 24, dtype=torch.float32) / 24))).to(DEV)
    out = torch.empty(6, 24, 2, device=DEV)
    ops.rope_table(pos, inv, out)
    ang = (inv[None, :] * pos.float()[:, None]).double()      # the float32 product, then exact functions
    assert (out[..., 0].double() - torch.cos(ang)).abs().max() < 3e-7
    assert (out[..., 1].double() - torch.sin(ang)).abs().max() < 3e-7


def _step(tok_seq, positions, tables):
    return types.SimpleNamespace(tok_seq=tok_seq, positions=positions, page_tables=[tables], is_decode=False,
                                 host_new=[], num_seqs=0, max_len=0)


def _cache(n_pages, nkv, hd, dtype):
    from hilbert_pruned_8b_b200.cache import LayerCache
    k = torch.zeros(n_pages, nkv, 64, hd, device=DEV, dtype=dtype)
    return LayerCache(k, torch.zeros_like(k), 0, None)


@pytest.mark.parametrize("nh,nkv,hd,rot,append", [(6, 3, 48, 48, True), (5, 1, 80, 32, True), (32, 8, 128, 128, True),
                                                  (3, 1, 64, 64, False)])
def test_rope_kv_append_many_tokens(ops, nh, nkv, hd, rot, append):
    """64 tokens and more take the one-block-per-token kernel with 16-byte accesses: the same
    bits as the few-token kernel (run here on slices of under 64 tokens)."""
    torch.manual_seed(33)
    lens = [70, 3, 130]                                     # three sequences, the first and last cross pages
    T = sum(lens)
    positions = torch.tensor([p for n in lens for p in range(n)], dtype=torch.int32, device=DEV)
    tok_seq = torch.tensor([i for i, n in enumerate(lens) for _ in range(n)], dtype=torch.int32, device=DEV)
    tables = torch.tensor([[5, 2, -1], [0, -1, -1], [1, 6, 3]], dtype=torch.int32, device=DEV)
    width = (nh + 2 * nkv) * hd
    qkv = torch.randn(T, width, device=DEV).to(torch.bfloat16)
    inv = (1.0 / (10000.0 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).to(DEV)
    table = torch.empty(T, rot // 2, 2, device=DEV)
    ops.rope_table(positions, inv, table)
    fast, cache_fast = qkv.clone(), _cache(7, nkv, hd, torch.bfloat16)
    ops.rope_kv_append(fast, table, rot, nh, nkv, hd, cache_fast, _step(tok_seq, positions, tables), append)
    slow, cache_slow = qkv.clone(), _cache(7, nkv, hd, torch.bfloat16)
    for a in range(0, T, 50):
        b = min(T, a + 50)
        ops.rope_kv_append(slow[a:b], table[a:b], rot, nh, nkv, hd, cache_slow, _step(tok_seq[a:b], positions[a:b], tables), append)
    assert torch.equal(fast, slow)
    assert torch.equal(cache_fast.k, cache_slow.k) and torch.equal(cache_fast.v, cache_slow.v)
    assert (cache_fast.k.abs().sum() > 0) == append
    assert cache_fast.k[4].abs().sum() == 0                 # a page of nobody stays clean


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,rot", [(6, 3, 48, 48), (5, 1, 80, 40), (8, 8, 16, 16)])
def test_rope_kv_append(ops, dtype, nh, nkv, hd, rot):
    torch.manual_seed(3)
    # two sequences: positions 60..69 (crossing a page) and 0..2; pages deliberately out of order
    positions = torch.tensor(list(range(60, 70)) + [0, 1, 2], dtype=torch.int32, device=DEV)
    tok_seq = torch.tensor([0] * 10 + [1] * 3, dtype=torch.int32, device=DEV)
    tables = torch.tensor([[5, 2], [0, -1]], dtype=torch.int32, device=DEV)
    T = 13
    width = (nh + 2 * nkv) * hd
    qkv = torch.randn(T, width, device=DEV).to(dtype)
    before = qkv.clone()
    cache = _cache(7, nkv, hd, dtype)
    inv = (1.0 / (10000.0 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).to(DEV)
    table = torch.empty(T, rot // 2, 2, device=DEV)
    ops.rope_table(positions, inv, table)
    ops.rope_kv_append(qkv, table, rot, nh, nkv, hd, cache, _step(tok_seq, positions, tables), True)

    def rotate(x):                                  # [T, heads, hd] in float64
        cs, sn = table[..., 0].double()[:, None, :], table[..., 1].double()[:, None, :]
        y = x.clone()
        h = rot // 2
        y[..., :h] = x[..., :h] * cs - x[..., h:rot] * sn
        y[..., h:rot] = x[..., h:rot] * cs + x[..., :h] * sn
        return y

    b = before.double()
    q_ref = rotate(b[:, :nh * hd].view(T, nh, hd))
    k_ref = rotate(b[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd))
    v_ref = b[:, (nh + nkv) * hd:].view(T, nkv, hd)
    tol = 1e-6 if dtype == torch.float32 else 2 ** -8
    assert _rel(qkv[:, :nh * hd].view(T, nh, hd), q_ref) < tol
    assert torch.equal(qkv[:, nh * hd:], before[:, nh * hd:])             # k and v columns untouched
    for t in range(T):
        page = int(tables[int(tok_seq[t]), int(positions[t]) // 64])
        off = int(positions[t]) % 64
        assert _rel(cache.k[page, :, off], k_ref[t]) < tol
        assert torch.equal(cache.v[page, :, off].double(), v_ref[t].to(dtype).double())
    assert cache.k.abs().sum(dim=(1, 3))[[1, 3, 4, 6]].sum() == 0          # pages of nobody stay clean
    # a layer that reads another layer's cache: only the queries turn, nothing is written
    qkv2, cache2 = before.clone(), _cache(7, nkv, hd, dtype)
    ops.rope_kv_append(qkv2, table, rot, nh, nkv, hd, cache2, _step(tok_seq, positions, tables), False)
    assert torch.equal(qkv2[:, :nh * hd], qkv[:, :nh * hd]) and cache2.k.abs().sum() == 0


# ------------------------------------------------------------------------------- matrix products
SHAPES = [(1, 128, 64), (8, 256, 160), (5, 100, 176), (33, 384, 416), (64, 512, 1024), (200, 300, 72), (300, 640, 256),
          (17, 129, 8), (2, 96, 4096)]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_general_float32(ops, M, N, K):
    torch.manual_seed(4)
    a, w = torch.randn(M, K, device=DEV), torch.randn(N, K, device=DEV)
    out = torch.full((M, N), 7.0, device=DEV)
    ops.linear(a, w, out)
    ref = a.double() @ w.double().t()
    assert _rel(out, ref) < 1e-6 * math.sqrt(K)
    res = torch.randn(M, N, device=DEV)
    acc = res.clone()
    ops.linear(a, w, acc, accumulate=True)
    assert _rel(acc, ref + res.double()) < 1e-6 * math.sqrt(K)


def test_gemm_general_mixed_dtypes_and_odd_k(ops):
    torch.manual_seed(5)
    a, w = _bf(torch.randn(9, 37, device=DEV)), torch.randn(50, 37, device=DEV)      # K = 37: no tensor-core path
    out = torch.empty(9, 50, device=DEV, dtype=torch.bfloat16)
    ops.linear(a, w, out)
    assert _rel(out, a.double() @ w.double().t()) < 2 ** -8
    a2, w2 = _bf(torch.randn(9, 37, device=DEV)), _bf(torch.randn(50, 37, device=DEV))
    out2 = torch.empty(9, 50, device=DEV)
    ops.linear(a2, w2, out2)
    assert _rel(out2, a2.double() @ w2.double().t()) < 1e-5


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_tensor_core_against_plain_and_general(ops, M, N, K):
    torch.manual_seed(6)
    a, w = _bf(torch.randn(M, K, device=DEV)), _bf(torch.randn(N, K, device=DEV))
    ref = a.double() @ w.double().t()
    for out_dtype in (torch.bfloat16, torch.float32):
        out = torch.full((M, N), 7.0, device=DEV, dtype=out_dtype)
        ops.linear(a, w, out)
        ops.check_errors()
        assert _rel(out, ref) < (2 ** -8 if out_dtype == torch.bfloat16 else 2e-6 * math.sqrt(K))
    res = torch.randn(M, N, device=DEV)
    acc = res.clone()
    ops.linear(a, w, acc, accumulate=True)
    ops.check_errors()
    assert _rel(acc, ref + res.double()) < 2e-6 * math.sqrt(K)
    # the general kernel on the same operands
    ops.use_tensor_cores = False
    try:
        gen = torch.empty(M, N, device=DEV)
        ops.linear(a, w, gen)
    finally:
        ops.use_tensor_cores = True
    out = torch.empty(M, N, device=DEV)
    ops.linear(a, w, out)
    assert _rel(out, gen) < 2e-6 * math.sqrt(K)


@pytest.mark.parametrize("M,N,K", [(8, 512, 1024), (1, 384, 4096), (64, 256, 2048), (5, 100, 416), (40, 4096, 512),
                                   (16, 20000, 256), (200, 384, 1024), (8, 28672, 512), (3, 19000, 64),
                                   (100, 512, 2048), (130, 4096, 1024), (256, 640, 4096), (300, 384, 2048)])
def test_gemm_tensor_core_stream_k_and_tiles(ops, M, N, K):
    """The work splits of the tensor-core kernel: stream-K (partial tiles in scratch, summed
    in K order by the last contributor), whole tiles round-robin (several per CTA), and cut
    tiles first with whole tiles after (what many tiles of few tokens get)."""
    torch.manual_seed(7)
    a, w = _bf(torch.randn(M, K, device=DEV)), _bf(torch.randn(N, K, device=DEV))
    ref = a.double() @ w.double().t()
    res = torch.randn(M, N, device=DEV)
    for schedule in ("stream_k", "tiles", "cut_first"):
        for rep in range(2):                    # twice: the tile counters must come back to zero
            acc = res.clone()
            ops.linear(a, w, acc, accumulate=True, schedule=schedule)
            ops.check_errors()
            assert _rel(acc, ref + res.double()) < 2e-6 * math.sqrt(K), schedule
        out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
        ops.linear(a, w, out, schedule=schedule)
        assert _rel(out, ref) < 2 ** -8
        assert int(ops._splitk_counters.abs().sum()) == 0
        again = torch.empty_like(out)
        ops.linear(a, w, again, schedule=schedule)
        assert torch.equal(out, again)          # the sum order is fixed


@pytest.mark.parametrize("M,N,K", [(512, 256, 64), (300, 640, 256), (1000, 1100, 520), (2048, 1024, 1024), (1, 128, 64),
                                   (257, 129, 72), (2600, 520, 128)])
def test_gemm_tensor_core_cta_pairs(ops, M, N, K):
    """The cta_group::2 kernel (256 x 256 tiles on pairs of CTAs) with every epilogue, at sizes
    with partial tiles in every dimension (2600 tokens: two groups of token tiles, the second
    short), against the plain product and the single-CTA kernel.  The epilogue writes whole
    tiles through shared memory (tile stores, tile adds) where the output's rows allow it and
    element by element where they do not: the two give the same bits."""
    torch.manual_seed(15)
    a, w = _bf(torch.randn(M, K, device=DEV)), _bf(torch.randn(N, K, device=DEV))
    ref = a.double() @ w.double().t()
    for out_dtype in (torch.bfloat16, torch.float32):
        out = torch.full((M, N), 7.0, device=DEV, dtype=out_dtype)
        ops.linear(a, w, out, schedule="pairs")
        ops.check_errors()
        assert _rel(out, ref) < (2 ** -8 if out_dtype == torch.bfloat16 else 2e-6 * math.sqrt(K))
    res = torch.randn(M, N, device=DEV)
    acc = res.clone()
    ops.linear(a, w, acc, accumulate=True, schedule="pairs")
    ops.check_errors()
    assert _rel(acc, ref + res.double()) < 2e-6 * math.sqrt(K)
    one = torch.empty(M, N, device=DEV)
    ops.linear(a, w, one, schedule="tiles")
    two = torch.empty(M, N, device=DEV)
    ops.linear(a, w, two, schedule="pairs")
    assert _rel(two, one) < 1e-6 * math.sqrt(K)
    assert ops.lib.hb_gemm_tc2_resident_pairs(0) >= 32
    # rows of N elements against rows a tile store cannot address (an odd stride) and rows it can
    for out_dtype, accumulate in ((torch.bfloat16, False), (torch.float32, False), (torch.float32, True)):
        results = []
        for pad in (0, 1, 8 - N % 8):
            wide = torch.full((M, N + pad), 3.0, device=DEV, dtype=out_dtype)
            view = wide[:, :N]
            if accumulate:
                view.copy_(res)
            ops.linear(a, w, view, accumulate=accumulate, schedule="pairs")
            ops.check_errors()
            assert pad == 0 or bool((wide[:, N:] == 3.0).all()), "the kernel wrote beside the output's rows"
            results.append(view.clone())
        assert torch.equal(results[0], results[1]) and torch.equal(results[0], results[2])


@pytest.mark.parametrize("M,N,K", [(8, 4096, 4096), (3, 3072, 3072), (16, 6144, 4096), (8, 2560, 2048), (8, 2304, 2112),
                                   (1, 4000, 1536), (32, 4096, 4096), (27, 2304, 2112), (64, 4096, 14336),
                                   (50, 3072, 3072), (64, 2560, 1024), (32, 2816, 1600), (64, 2816, 1600)])
def test_gemm_tensor_core_cluster_split(ops, M, N, K):
    """Up to 64 tokens and 19 to 74 tiles: every tile is cut into 2 to 8 K ranges whose CTAs
    form a cluster and sum their partial tiles over the first CTA's pipeline stages (K = 1536 and
    K = 1600 leave one CTA of each cluster without work).  Every epilogue, twice (same bits)."""
    torch.manual_seed(34)
    assert ops.lib.hb_gemm_tc_resident_clusters(2, 4) >= 32, "clusters of 4 do not fit: the cluster variant is not what runs here"
    a, w = _bf(torch.randn(M, K, device=DEV)), _bf(torch.randn(N, K, device=DEV))
    ref = a.double() @ w.double().t()
    res = torch.randn(M, N, device=DEV)
    acc = res.clone()
    ops.linear(a, w, acc, accumulate=True)
    ops.check_errors()
    assert _rel(acc, ref + res.double()) < 2e-6 * math.sqrt(K)
    acc2 = res.clone()
    ops.linear(a, ops.pack_weight(w), acc2, accumulate=True)
    assert torch.equal(acc, acc2)
    for dtype, tol in ((torch.bfloat16, 2 ** -8), (torch.float32, 2e-6 * math.sqrt(K))):
        out, again = torch.empty(M, N, device=DEV, dtype=dtype), torch.empty(M, N, device=DEV, dtype=dtype)
        ops.linear(a, w, out)
        ops.linear(a, w, again)
        ops.check_errors()
        assert _rel(out, ref) < tol and torch.equal(out, again)
    if N % 128 == 0:
        from hilbert_pruned_8b_b200.engine.workspace import Workspace
        I = N // 2
        act = torch.empty(M, I, device=DEV, dtype=torch.bfloat16)
        ws_ = _bf(w / math.sqrt(K))
        ops.linear_swiglu(a, ws_, act, Workspace(torch.device(DEV)), M)
        ops.check_errors()
        g, u = a.double() @ ws_[:I].double().t(), a.double() @ ws_[I:].double().t()
        assert _rel(act, g / (1 + torch.exp(-g)) * u) < 2 ** -7


@pytest.mark.parametrize("schedule", [None, "tiles", "stream_k", "cut_first"])
@pytest.mark.parametrize("M,H,K,I", [(8, 4096, 4096, 1024), (1, 2048, 8192, 512), (16, 264, 520, 192), (13, 3072, 1024, 256),
                                     (32, 2048, 2048, 640), (5, 1000, 320, 128), (23, 4096, 1024, 256)])
def test_norm_folded_into_the_products_around_it(ops, M, H, K, I, schedule):
    """Few tokens: the product that adds to the residual stream x also writes bf16(x * (offset + g))
    and partial sums of squares; the products that read that buffer multiply their rows by
    rsqrt(mean(x^2) + eps).  Against the plain statement in float64 and against the norm kernel
    followed by the plain products, in every work split of both sides (whole tiles, cut tiles,
    clusters) and every consumer epilogue (bfloat16, float32, SwiGLU)."""
    from hilbert_pruned_8b_b200.engine.workspace import Workspace
    torch.manual_seed(51)
    eps, offset = 1e-5, 0.25
    a = _bf(torch.randn(M, K, device=DEV))
    w = _bf(torch.randn(H, K, device=DEV) / math.sqrt(K))
    g = torch.randn(H, device=DEV) * 0.3 + 1.0
    x0 = torch.randn(M, H, device=DEV) * 3.0
    x0[M - 1] *= 40.0                                            # one token far larger than the others: the factor is per token
    w2 = _bf(torch.randn(2 * I, H, device=DEV) / math.sqrt(H))
    assert ops.can_fold_norm(M, H, torch.bfloat16)
    x = x0.clone()
    h = torch.full((M, H), 7.0, device=DEV, dtype=torch.bfloat16)
    prepared = ops.linear(a, w, x, accumulate=True, schedule=schedule, prepare=(g, offset, eps, h))
    ops.check_errors()
    assert prepared is not None
    # the residual itself: the same bits as without the preparation
    x_plain = x0.clone()
    ops.linear(a, w, x_plain, accumulate=True, schedule=schedule)
    assert torch.equal(x, x_plain)
    xd = x.double()
    assert torch.equal(h, _bf(x * (offset + g)))                 # the buffer: x * (offset + g), rounded once
    sums = prepared.sumsq[:M, :prepared.parts].double().sum(dim=1)
    assert ((sums - (xd * xd).sum(dim=1)).abs() / (xd * xd).sum(dim=1)).max() < 1e-6
    s = torch.rsqrt((xd * xd).mean(dim=1, keepdim=True) + eps)
    ref = (h.double() @ w2.double().t()) * s
    ws = Workspace(torch.device(DEV))
    for sched2 in (None, "tiles", "stream_k"):
        for dtype, tol in ((torch.bfloat16, 2 ** -8), (torch.float32, 2e-6 * math.sqrt(H))):
            y = torch.empty(M, 2 * I, device=DEV, dtype=dtype)
            ops.linear(h, w2, y, schedule=sched2, scale=prepared)
            ops.check_errors()
            assert _rel(y, ref) < tol, (sched2, dtype)
            worst = ((y.double() - ref).abs().amax(dim=1) / ref.abs().amax(dim=1)).max()
            assert worst < 4 * tol, f"a token's rows are off by {float(worst):.2e} of its own scale ({sched2}, {dtype})"
        act = torch.empty(M, I, device=DEV, dtype=torch.bfloat16)
        ops.linear_swiglu(h, w2, act, ws, M, schedule=sched2, scale=prepared)
        ops.check_errors()
        gate, up = ref[:, :I], ref[:, I:]
        want = gate / (1 + torch.exp(-gate)) * up
        assert ((act.double() - want).abs().amax(dim=1) / want.abs().amax(dim=1)).max() < 2 ** -6, sched2
    # against the norm kernel + plain products: the same up to the place of one rounding (bf16(x g s) there,
    # bf16(x g) s here).  Two independent bfloat16 roundings of every element of a row of H terms differ,
    # per output, by about 2^-9 of the row's scale; the largest of M * 2I such differences, as a fraction of
    # the row's largest output, comes to 0.0027-0.0037 at these sizes when both sides are computed in float64.
    hn = torch.empty(M, H, device=DEV, dtype=torch.bfloat16)
    ops.rmsnorm(x, g, eps, offset, hn)
    y1, y2 = torch.empty(M, 2 * I, device=DEV), torch.empty(M, 2 * I, device=DEV)
    ops.linear(hn, w2, y1)
    ops.linear(h, w2, y2, scale=prepared)
    assert ((y1 - y2).abs().amax(dim=1) / y1.abs().amax(dim=1)).max() < 2 ** -7
    with pytest.raises(Exception, match="does not scale"):
        ops.linear(a, w, x, accumulate=True, scale=prepared)
    # more tokens than the fold serves, or another dtype: the product says so and prepares nothing
    more = ops.FOLD_MAX_TOKENS + 1
    big = torch.zeros(more, H, device=DEV)
    assert ops.linear(_bf(torch.randn(more, K, device=DEV)), w, big, accumulate=True,
                      prepare=(g, offset, eps, torch.empty(more, H, device=DEV, dtype=torch.bfloat16))) is None


@pytest.mark.parametrize("M,N,K", [(8, 512, 1024), (5, 100, 416), (64, 300, 2048), (16, 1000, 72), (600, 640, 520)])
def test_gemm_tensor_core_packed_weights(ops, M, N, K):
    """A weight stored as contiguous 128 x 64 tiles gives bit for bit the results of the
    row-major one, in every work split and epilogue; a row prefix of it too; packing is exact."""
    from hilbert_pruned_8b_b200.kernels.ops import PackedWeight
    torch.manual_seed(31)
    a, w = _bf(torch.randn(M, K, device=DEV)), _bf(torch.randn(N, K, device=DEV))
    pw = PackedWeight.pack(w)
    assert pw.shape == (N, K) and torch.equal(pw.unpacked(), w)
    res = torch.randn(M, N, device=DEV)
    for schedule in ("stream_k", "tiles", "pairs"):
        for out_dtype in (torch.bfloat16, torch.float32):
            one, two = torch.empty(M, N, device=DEV, dtype=out_dtype), torch.empty(M, N, device=DEV, dtype=out_dtype)
            ops.linear(a, w, one, schedule=schedule)
            ops.linear(a, pw, two, schedule=schedule)
            ops.check_errors()
            assert torch.equal(one, two), (schedule, out_dtype)
        acc1, acc2 = res.clone(), res.clone()
        ops.linear(a, w, acc1, accumulate=True, schedule=schedule)
        ops.linear(a, pw, acc2, accumulate=True, schedule=schedule)
        assert torch.equal(acc1, acc2), schedule
    n = N - 37
    one, two = torch.empty(M, n, device=DEV), torch.empty(M, n, device=DEV)
    ops.linear(a, w[:n], one)
    ops.linear(a, pw.first_rows(n), two)
    assert torch.equal(one, two)
    ref = a.double() @ w.double().t()
    out = torch.empty(M, N, device=DEV)
    ops.linear(a, pw, out)
    assert _rel(out, ref) < 2e-6 * math.sqrt(K)


@pytest.mark.parametrize("M,K,I", [(3, 160, 448), (130, 256, 320), (8, 4096, 512), (700, 512, 1024)])
def test_linear_swiglu_packed_weights(ops, M, K, I):
    from hilbert_pruned_8b_b200.engine.workspace import Workspace
    torch.manual_seed(32)
    h = _bf(torch.randn(M, K, device=DEV))
    w = _bf(torch.randn(2 * I, K, device=DEV) / math.sqrt(K))
    pw = ops.pack_weight(w, swiglu=True)
    assert not isinstance(pw, torch.Tensor) and pw.gate_up_bands and torch.equal(pw.unpacked(), w)
    # band b: the gate rows of features 64 b .. 64 b + 63, then their up rows
    b = I // 64 - 1
    assert torch.equal(pw.data[b, 0, :64], w[64 * b:64 * b + 64, :64]) and torch.equal(pw.data[b, 0, 64:], w[I + 64 * b:I + 64 * b + 64, :64])
    with pytest.raises(Exception, match="linear_swiglu only"):
        ops.linear(h, pw, torch.empty(M, 2 * I, device=DEV))
    assert isinstance(ops.pack_weight(_bf(torch.randn(2 * 100, K, device=DEV)), swiglu=True), torch.Tensor)   # halves of 100 rows: not packed
    ws = Workspace(torch.device(DEV))
    for schedule in ("tiles", "stream_k", "pairs"):
        one, two = torch.empty(M, I, device=DEV, dtype=torch.bfloat16), torch.empty(M, I, device=DEV, dtype=torch.bfloat16)
        ops.linear_swiglu(h, w, one, ws, M, schedule=schedule)
        ops.linear_swiglu(h, pw, two, ws, M, schedule=schedule)
        ops.check_errors()
        assert torch.equal(one, two), schedule


@pytest.mark.parametrize("schedule", ["tiles", "stream_k", "pairs", "cut_first"])
@pytest.mark.parametrize("M,K,I", [(3, 160, 416), (40, 64, 176), (130, 256, 304), (8, 4096, 512), (300, 512, 1000), (1100, 192, 264)])
def test_linear_swiglu(ops, M, K, I, schedule):
    from hilbert_pruned_8b_b200.engine.workspace import Workspace
    torch.manual_seed(8)
    h = _bf(torch.randn(M, K, device=DEV))
    w = _bf(torch.randn(2 * I, K, device=DEV) / math.sqrt(K))
    act = torch.empty(M, I, device=DEV, dtype=torch.bfloat16)
    ws = Workspace(torch.device(DEV))
    ops.linear_swiglu(h, w, act, ws, M, schedule=schedule)
    ops.check_errors()
    g, u = h.double() @ w[:I].double().t(), h.double() @ w[I:].double().t()
    ref = g / (1 + torch.exp(-g)) * u
    assert _rel(act, ref) < 2 ** -7
    ops.use_tensor_cores = False
    try:
        slow = torch.empty_like(act)
        ops.linear_swiglu(h, w, slow, ws, M)
    finally:
        ops.use_tensor_cores = True
    assert _rel(slow, ref) < 2 ** -6     # the unfused path rounds gate and up to bfloat16 first


# ------------------------------------------------------------------------------- attention
def _attention_reference(q, keys, values, lens_before, new, nh, nkv, hd, scale, window):
    """q [T, nh, hd]; keys/values: per sequence [len, nkv, hd] float64."""
    out, t = [], 0
    for b, n in enumerate(new):
        for i in range(n):
            p = lens_before[b] + i
            lo = max(0, p - window + 1) if window else 0
            rows = []
            for j in range(nh):
                g = j // (nh // nkv)
                sc = (keys[b][lo:p + 1, g] @ q[t, j]) * scale
                rows.append(torch.softmax(sc, 0) @ values[b][lo:p + 1, g])
            out.append(torch.stack(rows))
            t += 1
    return torch.stack(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,window", [(6, 3, 48, None), (5, 1, 80, None), (4, 4, 16, 70), (8, 2, 128, None),
                                              (3, 1, 256, 33)])
def test_attention_general(ops, dtype, nh, nkv, hd, window):
    torch.manual_seed(9)
    lens_before, new = [130, 0, 63], [3, 70, 1]             # decode-like, prefill and a page edge in one batch
    total = [a + b for a, b in zip(lens_before, new)]
    keys = [torch.randn(n, nkv, hd, dtype=torch.float64) for n in total]
    values = [torch.randn(n, nkv, hd, dtype=torch.float64) for n in total]
    keys = [k.to(dtype).double() for k in keys]
    values = [v.to(dtype).double() for v in values]
    cache = _cache(9, nkv, hd, dtype)
    tables = torch.tensor([[7, 1, 4], [3, 8, -1], [0, -1, -1]], dtype=torch.int32, device=DEV)
    for b, n in enumerate(total):
        for s in range(n):
            page = int(tables[b, s // 64])
            cache.k[page, :, s % 64] = keys[b][s].to(dtype).to(DEV)
            cache.v[page, :, s % 64] = values[b][s].to(dtype).to(DEV)
    T = sum(new)
    q = torch.randn(T, nh, hd, dtype=torch.float64).to(dtype)
    qkv = torch.zeros(T, (nh + 2 * nkv) * hd, device=DEV, dtype=dtype)
    qkv[:, :nh * hd] = q.reshape(T, nh * hd).to(DEV)
    tok_seq = torch.tensor(sum(([b] * n for b, n in enumerate(new)), []), dtype=torch.int32, device=DEV)
    positions = torch.tensor(sum((list(range(l, l + n)) for l, n in zip(lens_before, new)), []), dtype=torch.int32,
                             device=DEV)
    out = torch.empty(T, nh * hd, device=DEV, dtype=dtype)
    scale = 1.0 / math.sqrt(hd)
    ops.use_fast_attention = False          # this test is about the general kernel
    try:
        ops.attention(qkv, nh, nkv, hd, cache, _step(tok_seq, positions, tables), out, scale, window)
    finally:
        ops.use_fast_attention = True
    ref = _attention_reference(q.double(), keys, values, lens_before, new, nh, nkv, hd, scale, window)
    assert _rel(out.view(T, nh, hd).cpu(), ref) < (2e-6 if dtype == torch.float32 else 2 ** -7)


@pytest.mark.parametrize("nh,nkv,hd,window", [(8, 2, 128, None), (3, 1, 64, None), (16, 1, 64, 100), (5, 5, 128, None),
                                              (12, 4, 128, 65)])
def test_attention_tensor_core_kernels(ops, nh, nkv, hd, window):
    """Split-K decode attention and flash prefill attention against the plain statement and the
    general kernel: a batch with lengths at page edges, several splits, a window."""
    torch.manual_seed(13)
    dtype = torch.bfloat16
    scale = 1.0 / math.sqrt(hd)
    for lens_before, new in (([130, 0, 63, 300], [1, 1, 1, 1]), ([130, 0, 63, 5], [3, 70, 1, 129])):
        total = [a + b for a, b in zip(lens_before, new)]
        keys = [torch.randn(n, nkv, hd, dtype=torch.float64).to(dtype).double() for n in total]
        values = [torch.randn(n, nkv, hd, dtype=torch.float64).to(dtype).double() for n in total]
        cache = _cache(16, nkv, hd, dtype)
        cache.k.normal_()            # stale contents of pages and page tails must not matter
        cache.v.normal_()
        tables = torch.tensor([[7, 1, 4, -1, -1], [3, 8, -1, -1, -1], [0, 15, -1, -1, -1], [9, 10, 11, 12, 13]],
                              dtype=torch.int32, device=DEV)
        for b, n in enumerate(total):
            for s0 in range(0, n, 64):
                page = int(tables[b, s0 // 64])
                seg = slice(s0, min(n, s0 + 64))
                cache.k[page, :, :seg.stop - s0] = keys[b][seg].to(dtype).transpose(0, 1).to(DEV)
                cache.v[page, :, :seg.stop - s0] = values[b][seg].to(dtype).transpose(0, 1).to(DEV)
        T = sum(new)
        q = torch.randn(T, nh, hd, dtype=torch.float64).to(dtype)
        qkv = torch.zeros(T, (nh + 2 * nkv) * hd, device=DEV, dtype=dtype)
        qkv[:, :nh * hd] = q.reshape(T, nh * hd).to(DEV)
        step = _step(torch.tensor(sum(([b] * n for b, n in enumerate(new)), []), dtype=torch.int32, device=DEV),
                     torch.tensor(sum((list(range(l, l + n)) for l, n in zip(lens_before, new)), []), dtype=torch.int32,
                                  device=DEV), tables)
        starts = [0]
        for n in new:
            starts.append(starts[-1] + n)
        step.seq_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
        step.seq_pos0 = torch.tensor(lens_before, dtype=torch.int32, device=DEV)
        step.is_decode = all(n == 1 for n in new)
        step.host_new, step.num_seqs, step.max_len = new, len(new), max(total)
        ref = _attention_reference(q.double(), keys, values, lens_before, new, nh, nkv, hd, scale, window)
        for splits in ((None, 1, 3) if step.is_decode else (None,)):
            out = torch.full((T, nh * hd), 9.0, device=DEV, dtype=dtype)
            ops.attention(qkv, nh, nkv, hd, cache, step, out, scale, window, splits=splits)
            ops.check_errors()
            assert _rel(out.view(T, nh, hd).cpu(), ref) < 2 ** -7, f"splits={splits} decode={step.is_decode}"
            if step.is_decode:                 # a second kernel combined above; now the last split does
                ops.combine_in_attention = True
                try:
                    two = torch.full((T, nh * hd), 9.0, device=DEV, dtype=dtype)
                    ops.attention(qkv, nh, nkv, hd, cache, step, two, scale, window, splits=splits)
                finally:
                    ops.combine_in_attention = False
                assert _rel(two.view(T, nh, hd).cpu(), ref) < 2 ** -7
                assert int(ops._decode_counters.abs().sum()) == 0
        if not step.is_decode:                 # the tcgen05 kernel ran above; now the mma.sync one
            ops.use_tcgen05_attention = False
            try:
                other = torch.full((T, nh * hd), 9.0, device=DEV, dtype=dtype)
                ops.attention(qkv, nh, nkv, hd, cache, step, other, scale, window)
            finally:
                ops.use_tcgen05_attention = True
            assert _rel(other.view(T, nh, hd).cpu(), ref) < 2 ** -7
        ops.use_fast_attention = False
        try:
            gen = torch.empty(T, nh * hd, device=DEV, dtype=dtype)
            ops.attention(qkv, nh, nkv, hd, cache, step, gen, scale, window)
        finally:
            ops.use_fast_attention = True
        assert _rel(out, gen.double()) < 2 ** -7


@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 128, None), (6, 2, 64, None), (4, 1, 128, 300), (2, 2, 64, 65),
                                              (2, 1, 128, 128)])
def test_attention_prefill_long_prompts(ops, nh, nkv, hd, window):
    """The tcgen05 prefill kernel on prompts of several query tiles and many key tiles: full and
    short last tiles, new tokens behind a long context that starts inside a key tile, windows
    shorter and longer than a tile, pages in a shuffled order.  One key of the longest prompt is
    made to stand out for one query far behind it."""
    torch.manual_seed(41)
    dtype = torch.bfloat16
    scale = 1.0 / math.sqrt(hd)
    lens_before, new = [100, 0, 64, 1000, 0], [257, 600, 128, 5, 384]
    total = [a + b for a, b in zip(lens_before, new)]
    keys = [torch.randn(n, nkv, hd, device=DEV).to(dtype) for n in total]
    values = [torch.randn(n, nkv, hd, device=DEV).to(dtype) for n in total]
    T = sum(new)
    q = torch.randn(T, nh, hd, device=DEV).to(dtype)
    # sequence 1 (600 new tokens from position 0): query 570 of head nh - 1 looks for key 9
    needle_q, needle_k = new[0] + 570, 9
    keys[1][needle_k, nkv - 1] = 2.0
    q[needle_q, nh - 1] = 4.0
    pages_of = [(n + 63) // 64 for n in total]
    n_pages = sum(pages_of) + 3
    order = torch.randperm(n_pages).tolist()
    tables = torch.full((len(total), max(pages_of) + 1), -1, dtype=torch.int32)
    cache = _cache(n_pages, nkv, hd, dtype)
    cache.k.normal_()
    cache.v.normal_()
    for b, n in enumerate(total):
        for i in range(pages_of[b]):
            page = order.pop()
            tables[b, i] = page
            seg = slice(64 * i, min(n, 64 * i + 64))
            cache.k[page, :, :seg.stop - seg.start] = keys[b][seg].transpose(0, 1)
            cache.v[page, :, :seg.stop - seg.start] = values[b][seg].transpose(0, 1)
    tables = tables.to(DEV)
    qkv = torch.zeros(T, (nh + 2 * nkv) * hd, device=DEV, dtype=dtype)
    qkv[:, :nh * hd] = q.reshape(T, nh * hd)
    step = _step(torch.tensor(sum(([b] * n for b, n in enumerate(new)), []), dtype=torch.int32, device=DEV),
                 torch.tensor(sum((list(range(l, l + n)) for l, n in zip(lens_before, new)), []), dtype=torch.int32, device=DEV),
                 tables)
    starts = [0]
    for n in new:
        starts.append(starts[-1] + n)
    step.seq_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
    step.seq_pos0 = torch.tensor(lens_before, dtype=torch.int32, device=DEV)
    step.host_new, step.num_seqs, step.max_len = new, len(new), max(total)
    out = torch.full((T, nh * hd), 9.0, device=DEV, dtype=dtype)
    ops.call_log = []
    try:
        ops.attention(qkv, nh, nkv, hd, cache, step, out, scale, window)
        ops.check_errors()
        assert "hb_attention_prefill_tc" in ops.call_log
    finally:
        ops.call_log = None
    # the plain statement in float64 on the device, sequence by sequence
    group = nh // nkv
    for b, n in enumerate(new):
        qb = q[starts[b]:starts[b + 1]].double()                                   # [n, nh, hd]
        kb = keys[b].double().repeat_interleave(group, dim=1)                        # [total, nh, hd]
        vb = values[b].double().repeat_interleave(group, dim=1)
        sc = torch.einsum("qhd,khd->hqk", qb, kb) * scale
        pos = torch.arange(lens_before[b], lens_before[b] + n, device=DEV).view(1, n, 1)
        kpos = torch.arange(total[b], device=DEV).view(1, 1, -1)
        seen = kpos <= pos
        if window:
            seen = seen & (kpos > pos - window)
        ref = torch.einsum("hqk,khd->qhd", torch.softmax(sc.masked_fill(~seen, float("-inf")), dim=-1), vb)
        got = out[starts[b]:starts[b + 1]].view(n, nh, hd).double()
        assert _rel(got, ref) < 2 ** -7, f"sequence {b}"
        worst = (got - ref).abs().amax(dim=(1, 2))
        assert worst.max() < 0.05, f"sequence {b}: row {int(worst.argmax())} is off by {float(worst.max()):.3f}"
    if window is None:
        far = out[needle_q].view(nh, hd)[nh - 1].float()
        assert (far - values[1][needle_k, nkv - 1].float()).abs().max() < 0.03


def test_decode_attention_split_choice(ops):
    """The number of key splits: one wave of CTAs that fills the device where there is one, whole
    waves where one split per (sequence, kv head) would leave a third of a wave idle, never
    more than a split for every eight pages, never more than 16 splits."""
    per_sm = ops.lib.hb_attention_decode_ctas_per_sm(128)
    assert per_sm >= 1 and ops.lib.hb_attention_decode_ctas_per_sm(64) >= per_sm and ops.lib.hb_attention_decode_ctas_per_sm(80) == 0
    slots = ops.sm_count * per_sm
    for batch, kv, pages in [(1, 8, 128), (8, 8, 128), (8, 8, 4), (24, 8, 128), (48, 8, 128), (64, 8, 128), (3, 1, 1000), (500, 8, 40)]:
        s = ops.decode_splits_for(batch, kv, pages, 128)
        assert 1 <= s <= 16 and s <= -(-pages // 8), (batch, kv, pages, s)
        ctas = batch * kv * s
        if batch * kv <= slots // 2 and pages >= 16 * (slots // (batch * kv)):
            assert ctas > slots // 2 or s == 16, (batch, kv, pages, s)           # few sequences with long caches fill the device
    if ops.sm_count == 148 and per_sm == 2:
        assert [ops.decode_splits_for(b, 8, 128, 128) for b in (8, 16, 32, 48, 64)] == [4, 2, 1, 2, 1]


@pytest.mark.parametrize("nh,nkv,hd,rot,window,copies", [(8, 2, 128, 128, None, 1), (3, 1, 64, 64, None, 1),
                                                         (16, 1, 64, 32, 100, 1), (10, 5, 128, 128, 65, 1),
                                                         (8, 4, 128, 128, None, 14), (8, 2, 64, 64, 100, 32)])
def test_attention_decode_fused_equals_the_three_kernels(ops, nh, nkv, hd, rot, window, copies):
    """The decode attention that rotates and appends itself (with the combination kernel behind
    it, or combining in its last split) against the separate rope/append, attention and combine
    kernels, twice in a row (counters return to zero), with lengths at page edges and a first
    token.  Few sequences run the deep page pipeline (a CTA per SM at most), `copies` of them
    the shallow one."""
    torch.manual_seed(14)
    dtype = torch.bfloat16
    scale = 1.0 / math.sqrt(hd)
    positions = [130, 0, 63, 300, 64] * copies
    B = len(positions)
    rows = [[7, 1, 4, -1, -1], [3, 8, -1, -1, -1], [0, 15, -1, -1, -1], [9, 10, 11, 12, 13], [2, 5, -1, -1, -1]]
    tables = torch.tensor([[p + 16 * c if p >= 0 else -1 for p in row] for c in range(copies) for row in rows],
                          dtype=torch.int32, device=DEV)
    base = _cache(16 * copies, nkv, hd, dtype)
    base.k.normal_()
    base.v.normal_()
    step = _step(torch.arange(B, dtype=torch.int32, device=DEV), torch.tensor(positions, dtype=torch.int32, device=DEV), tables)
    step.is_decode, step.host_new, step.num_seqs, step.num_tokens = True, [1] * B, B, B
    step.max_len = max(positions) + 1
    step.seq_start = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    step.seq_pos0 = step.positions
    inv = (1.0 / (10000.0 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).to(DEV)
    table = torch.empty(B, rot // 2, 2, device=DEV)
    ops.rope_table(step.positions, inv, table)
    for rep in range(2):
        qkv = torch.randn(B, (nh + 2 * nkv) * hd, device=DEV).to(dtype)
        from hilbert_pruned_8b_b200.cache import LayerCache
        c1 = LayerCache(base.k.clone(), base.v.clone(), 0, None)
        c2 = LayerCache(base.k.clone(), base.v.clone(), 0, None)
        q1 = qkv.clone()
        ops.rope_kv_append(q1, table, rot, nh, nkv, hd, c1, step, True)
        want = torch.empty(B, nh * hd, device=DEV, dtype=dtype)
        ops.attention(q1, nh, nkv, hd, c1, step, want, scale, window)
        for splits in (None, 1, 3):
            c3 = LayerCache(c2.k.clone(), c2.v.clone(), 0, None)
            got = torch.full_like(want, 9.0)
            before = qkv.clone()
            assert ops.can_fuse_decode_attention(qkv, nh, nkv, hd, c3, step, got)
            for inside in (False, True):          # a combination kernel, or the last split combines
                c3.k.copy_(c2.k)
                c3.v.copy_(c2.v)
                got.fill_(9.0)
                ops.combine_in_attention = inside
                try:
                    ops.attention_decode_fused(qkv, table, rot, nh, nkv, hd, c3, step, got, scale, window, True, splits=splits)
                finally:
                    ops.combine_in_attention = False
                assert torch.equal(qkv, before)
                assert torch.equal(c3.k, c1.k) and torch.equal(c3.v, c1.v), "appended keys or values differ"
                assert _rel(got, want.double()) < 2 ** -8, f"splits={splits} inside={inside}"
        assert int(ops._decode_counters.abs().sum()) == 0
    # a layer that reads another layer's cache: no append, the new key is not there
    c4 = LayerCache(base.k.clone(), base.v.clone(), 0, None)
    got = torch.empty(B, nh * hd, device=DEV, dtype=dtype)
    ops.attention_decode_fused(qkv, table, rot, nh, nkv, hd, c4, step, got, scale, window, False)
    assert torch.equal(c4.k, base.k) and torch.equal(c4.v, base.v)
    q1 = qkv.clone()
    ops.rope_kv_append(q1, table, rot, nh, nkv, hd, c4, step, False)
    want = torch.empty_like(got)
    ops.attention(q1, nh, nkv, hd, c4, step, want, scale, window)
    assert _rel(got, want.double()) < 2 ** -8


@pytest.mark.parametrize("hd,dtype", [(32, torch.float32), (128, torch.bfloat16), (64, torch.bfloat16)])
def test_attention_finds_a_far_key(ops, hd, dtype):
    """One key among hundreds matches the query: the output must be that key's value (general
    kernel for head size 32, the split-K decode kernel for 64 and 128)."""
    nh, nkv, n = 4, 2, 700
    torch.manual_seed(10)
    cache = _cache(12, nkv, hd, dtype)
    tables = torch.arange(11, -1, -1, dtype=torch.int32, device=DEV).view(1, 12)
    k = torch.randn(n, nkv, hd) * 0.1
    v = torch.randn(n, nkv, hd)
    needle = 137
    k[needle, 1] = torch.ones(hd) * 3.0
    v = v.to(dtype).float()
    for s in range(n):
        cache.k[int(tables[0, s // 64]), :, s % 64] = k[s].to(dtype).to(DEV)
        cache.v[int(tables[0, s // 64]), :, s % 64] = v[s].to(dtype).to(DEV)
    qkv = torch.zeros(1, (nh + 2 * nkv) * hd, device=DEV, dtype=dtype)
    qkv[0, 3 * hd:4 * hd] = 10.0                                   # head 3 reads kv head 1
    out = torch.empty(1, nh * hd, device=DEV, dtype=dtype)
    step = _step(torch.zeros(1, dtype=torch.int32, device=DEV), torch.tensor([n - 1], dtype=torch.int32, device=DEV), tables)
    step.is_decode, step.host_new, step.num_seqs, step.max_len, step.num_tokens = True, [1], 1, n, 1
    ops.attention(qkv, nh, nkv, hd, cache, step, out, 1.0 / math.sqrt(hd), None)
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert (out[0, 3 * hd:].float().cpu() - v[needle, 1]).abs().max() < tol
    assert (out[0, :hd].float().cpu() - v[:, 0].mean(0)).abs().max() < tol   # a zero query averages the values


# ------------------------------------------------------------------------------- sampling
@pytest.mark.parametrize("vocab", [7, 384, 5003, 128256])
def test_argmax_lowest_index_on_ties(ops, vocab):
    torch.manual_seed(11)
    lg = torch.randn(5, vocab, device=DEV)
    lg[1, vocab - 1] = 9.0
    lg[2, 3] = lg[2, vocab // 2] = 11.0
    lg[3] = 0.0
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    ops.argmax(lg, out)
    want = [int(lg[0].argmax()), vocab - 1, 3, 0, int(lg[4].argmax())]
    assert out.tolist() == want


@pytest.mark.parametrize("rows", [1, 8, 40, 300])
def test_argmax_rows_cut_over_several_blocks(ops, rows):
    """With few rows each row is cut into ranges for several blocks (the last one to finish takes
    the best of them): the lowest index still wins a tie across ranges, the counters come back
    to zero (twice in a row), rows whose storage is not 16-byte aligned work too."""
    torch.manual_seed(13 + rows)
    vocab = 128256
    lg = torch.randn(rows, vocab, device=DEV)
    lg[0, 100000] = lg[0, 20] = lg[0, 64200] = 30.0             # a tie across ranges
    if rows > 1:
        lg[1, vocab - 1] = 31.0
        lg[rows - 1] = -5.0                                        # a constant row: index 0
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    for _ in range(2):
        out.fill_(-1)
        ops.argmax(lg, out)
        assert out[0].item() == 20 and torch.equal(out[1:].long(), lg[1:].argmax(dim=1))
        assert int(ops._argmax_counters.abs().sum()) == 0
    odd = torch.randn(3, vocab + 3, device=DEV)[:, 3:]
    out3 = torch.empty(3, dtype=torch.int32, device=DEV)
    ops.argmax(odd, out3)
    assert torch.equal(out3.long(), odd.argmax(dim=1))
    assert ops.status.tolist() == [0, 0, 0, 0]


@pytest.mark.parametrize("vocab", [11, 384, 50257])
def test_temperature_sampling_follows_the_cdf(ops, vocab):
    from hilbert_pruned_8b_b200.sampling import uniform_from
    torch.manual_seed(12)
    n = 64
    lg = torch.randn(n, vocab, device=DEV) * 2
    temps = [0.8] * (n - 2) + [0.0, 1.7]
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    seeds = torch.full((n,), 1234, dtype=torch.int64, device=DEV)
    reqs = torch.arange(n, dtype=torch.int64, device=DEV)
    steps = torch.full((n,), 5, dtype=torch.int64, device=DEV)
    ops.sample(lg, torch.tensor(temps, device=DEV), seeds, reqs, steps, out)
    got = out.tolist()
    for r in range(n):
        if temps[r] == 0.0:
            assert got[r] == int(lg[r].argmax())
            continue
        p = torch.softmax(lg[r].double().cpu() / temps[r], 0)
        c = torch.cumsum(p, 0)
        u = uniform_from(1234, r, 5)
        lo = float(c[got[r] - 1]) if got[r] > 0 else 0.0
        assert lo - 1e-5 <= u <= float(c[got[r]]) + 1e-5, f"row {r}: u={u} outside the chosen token's interval"
    again = torch.empty_like(out)
    ops.sample(lg, torch.tensor(temps, device=DEV), seeds, reqs, steps, again)
    assert torch.equal(out, again)
    ops.sample(lg, torch.tensor(temps, device=DEV), seeds, reqs, steps + 1, again)
    assert not torch.equal(out, again)
