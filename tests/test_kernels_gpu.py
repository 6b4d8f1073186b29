"""Each kernel alone against a plain PyTorch float32 reference of the same
operation, at sizes other than the engine tests use: widths and vocabularies
that are no power of two, every head size in steps of 16, ragged batches, pages
scattered over the cache, and inputs made so that a wrong key shows."""
import math

import numpy as np
import pytest
import torch

import go_tinygrad_b200  # noqa: F401
from go_tinygrad_b200.cache import Cache, KVRequest
from go_tinygrad_b200.kernels import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


# ------------------------------------------------------------------ elementwise
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,V,N", [(24, 37, 5), (2048, 1000, 33), (1000, 129, 7)])
def test_embed(dtype, H, V, N):
    table = rnd(V, H, dtype=dtype)
    tokens = torch.randint(0, V, (N,), dtype=torch.int32, device=DEV)
    tokens[0], tokens[-1] = V - 1, 0
    out = torch.empty(N, H, dtype=torch.float32, device=DEV)
    ops.embed(tokens, table, out)
    assert torch.equal(out, table[tokens.long()].float())


def ref_rmsnorm(x, w, eps):
    return w * x * torch.rsqrt((x.double() ** 2).mean(-1, keepdim=True) + eps).float()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,N,eps", [(24, 3, 1e-5), (2048, 19, 1e-6), (1000, 4, 1e-3), (13000, 2, 1e-5), (36, 5, 1e-5),
                                     (8192, 3, 1e-5),
                                     # many rows (a prompt)
                                     (2048, 300, 1e-5), (1000, 257, 1e-6), (264, 1001, 1e-5), (1024, 256, 1e-5),
                                     (1032, 260, 1e-5), (4096, 300, 1e-5), (40, 2048, 1e-5)])
def test_add_rmsnorm(dtype, H, N, eps):
    res = rnd(N, H, scale=3.0, seed=1)
    pend = rnd(N, H, dtype=dtype, seed=2)
    w = 1 + 0.1 * rnd(H, seed=3)
    # with a pending update: the sum lands in the residual
    r1 = res.clone()
    out = torch.empty(N, H, dtype=dtype, device=DEV)
    ops.add_rmsnorm(r1, pend, w, eps, out)
    summed = res + pend.float()
    torch.testing.assert_close(r1, summed, rtol=0, atol=0)
    torch.testing.assert_close(out.float(), ref_rmsnorm(summed, w, eps).to(dtype).float(), **tol(dtype))
    # without one: the residual is untouched
    r2 = res.clone()
    ops.add_rmsnorm(r2, None, w, eps, out)
    assert torch.equal(r2, res)
    torch.testing.assert_close(out.float(), ref_rmsnorm(res, w, eps).to(dtype).float(), **tol(dtype))
    # selected rows: nothing is written back, rows may repeat
    rows = torch.tensor([N - 1, 0, N - 1], dtype=torch.int32, device=DEV)
    r3 = res.clone()
    out3 = torch.empty(3, H, dtype=dtype, device=DEV)
    ops.add_rmsnorm(r3, pend, w, eps, out3, rows)
    assert torch.equal(r3, res)
    torch.testing.assert_close(out3.float(), ref_rmsnorm(summed[rows.long()], w, eps).to(dtype).float(),
                               **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,I", [(1, 8), (7, 264), (130, 1000)])
def test_swiglu(dtype, M, I):
    gu = rnd(M, 2 * I, dtype=dtype, scale=3.0)
    out = torch.empty(M, I, dtype=dtype, device=DEV)
    ops.swiglu(gu, out)
    g, u = gu[:, :I].float(), gu[:, I:].float()
    want = (g / (1 + torch.exp(-g)) * u).to(dtype).float()
    torch.testing.assert_close(out.float(), want, **tol(dtype))


def test_rope_table_is_float64_accurate():
    half = 24
    inv = torch.tensor([1.0 / math.pow(500000.0, 2 * i / (2 * half)) for i in range(half)],
                       dtype=torch.float64, device=DEV)
    pos = torch.tensor([0, 1, 63, 64, 8191, 131071, 1 << 24], dtype=torch.int32, device=DEV)
    out = torch.empty(pos.numel(), half, 2, dtype=torch.float32, device=DEV)
    ops.rope_table(pos, inv, out)
    ang = pos.double().cpu()[:, None] * inv.cpu()[None, :]
    want = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).float()
    # float rounding of a correctly computed value only: an angle formed in float32
    # would be off by up to 1e-3 at these positions
    torch.testing.assert_close(out.cpu(), want, rtol=0, atol=2e-7)


def make_cache(n_kv, hd, dtype, n_pages=40, n_entries=2, window=None):
    """A cache with one group whose pages are handed out in a scrambled order, so
    that a kernel that ignored the block table would read the wrong memory."""
    cache = Cache([[KVRequest(n_kv, hd, window)] for _ in range(n_entries)], [None] * n_entries,
                  max_tokens=n_pages * 64, max_slots=8, dtype=dtype, device=DEV)
    pool = cache.groups[0].pool
    rng = np.random.default_rng(5)
    pool._free = [int(p) for p in rng.permutation(n_pages)]
    return cache


def fill_sequence(cache, entry, slot, k, v):
    """Write k, v [T, n_kv, hd] as the first T tokens of `slot` (test-side scatter)."""
    T = k.shape[0]
    cache.reserve(slot, T)
    cache.flush_tables()
    view = cache.handles[entry].kv
    t = torch.arange(T)
    pages = cache.groups[0].table_host[slot][t // 64].long().to(DEV)
    view.k[pages, :, (t % 64).to(DEV), :] = k
    view.v[pages, :, (t % 64).to(DEV), :] = v
    cache._length[slot] = T


def read_sequence(cache, entry, slot, T):
    view = cache.handles[entry].kv
    t = torch.arange(T)
    pages = cache.groups[0].table_host[slot][t // 64].long().to(DEV)
    k = view.k[pages, :, (t % 64).to(DEV), :]
    v = view.v[pages, :, (t % 64).to(DEV), :]
    return k, v


@pytest.mark.parametrize("n_heads,n_kv,K", [(8, 8, 256), (6, 2, 520), (3, 1, 64), (32, 8, 2048)])
def test_qkv_projection_with_rotation_and_cache_store_in_its_epilogue(n_heads, n_kv, K):
    """linear_qkv_rope against the plain product followed by the plain rotation:
    rotated queries in the output, rotated keys and values in the cache at each
    token's (slot, position), other cache entries and pages untouched."""
    hd, dtype = 64, torch.bfloat16
    cache = make_cache(n_kv, hd, dtype)
    slots = [cache.open_sequence() for _ in range(3)]
    starts, lens = [0, 61, 130], [70, 129, 3]     # runs that cross page borders; 202 rows: two row tiles
    for s, st, n in zip(slots, starts, lens):
        cache.reserve(s, st + n)
        cache._length[s] = st
    cache.flush_tables()
    N, width = sum(lens), (n_heads + 2 * n_kv) * hd
    x = rnd(N, K, dtype=dtype, seed=3, scale=0.5)
    w = rnd(width, K, dtype=dtype, seed=4, scale=0.2)
    positions = torch.tensor([st + j for st, n in zip(starts, lens) for j in range(n)], dtype=torch.int32, device=DEV)
    token_seq = torch.tensor([b for b, n in enumerate(lens) for _ in range(n)], dtype=torch.int32, device=DEV)
    slot_t = torch.tensor(slots, dtype=torch.int32, device=DEV)
    inv = torch.tensor([1.0 / math.pow(10000.0, 2 * i / hd) for i in range(32)], dtype=torch.float64, device=DEV)
    cs = torch.empty(N, 32, 2, dtype=torch.float32, device=DEV)
    ops.rope_table(positions, inv, cs)
    kv = cache.handles[1].kv
    qkv = torch.full((N, width), 7.0, dtype=dtype, device=DEV)
    assert ops.qkv_rope_fused_supports(x, w, qkv, cs, n_heads, n_kv, hd, kv)
    ops.linear_qkv_rope(x, w, qkv, cs, n_heads, n_kv, kv, token_seq, slot_t, positions)
    assert ops.bounded_wait_failures() == 0

    full = x.double() @ w.double().T

    def rot(t, nh):
        t = t.reshape(N, nh, hd)
        a, b = t[..., :32], t[..., 32:]
        c, s = cs[:, None, :, 0].double(), cs[:, None, :, 1].double()
        return torch.cat([a * c - b * s, a * s + b * c], dim=-1)
    scale = float(full.abs().max())
    want_q = rot(full[:, : n_heads * hd], n_heads).reshape(N, -1).float()
    want_k = rot(full[:, n_heads * hd: (n_heads + n_kv) * hd], n_kv).float()
    want_v = full[:, (n_heads + n_kv) * hd:].reshape(N, n_kv, hd).float()
    close = dict(rtol=1.6e-2, atol=1e-2 * max(1.0, scale / 4))
    torch.testing.assert_close(qkv[:, : n_heads * hd].float(), want_q, **close)
    assert float((qkv[:, n_heads * hd:].float() - 7.0).abs().sum()) == 0.0    # key and value columns are not written
    o = 0
    for s, st, n in zip(slots, starts, lens):
        k, v = read_sequence(cache, 1, s, st + n)
        torch.testing.assert_close(k[st:].float(), want_k[o:o + n], **close)
        torch.testing.assert_close(v[st:].float(), want_v[o:o + n], **close)
        assert float(k[:st].abs().sum()) == 0.0            # nothing written before the run
        o += n
    assert float(cache.handles[0].kv.k.abs().sum()) == 0.0  # the other entry is untouched


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_heads,n_kv,hd", [(4, 2, 16), (3, 1, 48), (8, 8, 64), (5, 5, 112), (2, 2, 24), (32, 8, 128)])
def test_rope_kv_store(dtype, n_heads, n_kv, hd):
    cache = make_cache(n_kv, hd, dtype)
    slots = [cache.open_sequence() for _ in range(3)]
    starts, lens = [0, 61, 130], [5, 9, 3]       # runs that cross page borders
    for s, st in zip(slots, starts):
        cache.reserve(s, st + 70)
        cache._length[s] = st
    cache.flush_tables()
    N = sum(lens)
    width = (n_heads + 2 * n_kv) * hd + 8          # a row stride wider than the data
    buf = rnd(N, width, dtype=dtype, seed=7)
    qkv = buf[:, : (n_heads + 2 * n_kv) * hd]
    before = qkv.clone()
    positions = torch.tensor([st + j for st, n in zip(starts, lens) for j in range(n)], dtype=torch.int32, device=DEV)
    token_seq = torch.tensor([b for b, n in enumerate(lens) for _ in range(n)], dtype=torch.int32, device=DEV)
    slot_t = torch.tensor(slots, dtype=torch.int32, device=DEV)
    half = hd // 2
    inv = torch.tensor([1.0 / math.pow(10000.0, 2 * i / hd) for i in range(half)], dtype=torch.float64, device=DEV)
    cs = torch.empty(N, half, 2, dtype=torch.float32, device=DEV)
    ops.rope_table(positions, inv, cs)
    ops.rope_kv_store(qkv, cs, n_heads, n_kv, hd, cache.handles[1].kv, token_seq, slot_t, positions)

    def rot(x, nh):
        x = x.float().reshape(N, nh, hd)
        a, b = x[..., :half], x[..., half:]
        c, s = cs[:, None, :, 0], cs[:, None, :, 1]
        return torch.cat([a * c - b * s, a * s + b * c], dim=-1).to(dtype)
    want_q = rot(before[:, : n_heads * hd], n_heads).reshape(N, -1)
    want_k = rot(before[:, n_heads * hd: (n_heads + n_kv) * hd], n_kv)
    want_v = before[:, (n_heads + n_kv) * hd:].reshape(N, n_kv, hd)
    torch.testing.assert_close(qkv[:, : n_heads * hd].float(), want_q.float(), **tol(dtype))
    assert torch.equal(qkv[:, n_heads * hd:], before[:, n_heads * hd:])      # k, v columns untouched
    assert torch.equal(buf[:, -8:], rnd(N, width, dtype=dtype, seed=7)[:, -8:])
    o = 0
    for s, st, n in zip(slots, starts, lens):
        k, v = read_sequence(cache, 1, s, st + n)
        torch.testing.assert_close(k[st:].float(), want_k[o:o + n].float(), **tol(dtype))
        assert torch.equal(v[st:], want_v[o:o + n])
        assert float(k[:st].abs().sum()) == 0.0            # nothing written before the run
        o += n
    assert float(cache.handles[0].kv.k.abs().sum()) == 0.0  # the other entry is untouched


# -------------------------------------------------------------- matrix products
@pytest.mark.parametrize("M,N,K", [(1, 17, 8), (5, 96, 264), (64, 391, 96), (130, 130, 40),
                                   (257, 1000, 2048), (3, 2048, 8192)])
def test_linear_float32(M, N, K):
    x, w = rnd(M, K, seed=1), rnd(N, K, seed=2)
    out = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.linear(x, w, out)
    want = (x.double() @ w.double().T).float()
    torch.testing.assert_close(out, want, rtol=1e-5, atol=1e-4 * math.sqrt(K / 64))


def test_linear_float32_does_not_depend_on_the_batch():
    """A row's result is bitwise the same alone, in a small batch, in a large one."""
    K, N = 264, 391
    x, w = rnd(200, K, seed=1), rnd(N, K, seed=2)
    full = torch.empty(200, N, dtype=torch.float32, device=DEV)
    ops.linear(x, w, full)
    for rows in ([0], [63, 64], list(range(100, 177))):
        sub = x[rows].contiguous()
        out = torch.empty(len(rows), N, dtype=torch.float32, device=DEV)
        ops.linear(sub, w, out)
        assert torch.equal(out, full[rows])


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("kind", ["skinny", "swapab", "tiled", "tcgen05"])
@pytest.mark.parametrize("M,N,K", [(1, 17, 8), (5, 96, 264), (64, 391, 96), (130, 130, 40),
                                   (257, 1000, 2048), (3, 2048, 8192), (8, 6144, 2048),
                                   (300, 144, 96), (9, 50, 1000), (17, 33, 72), (40, 1001, 2056),
                                   (33, 16, 8200), (65, 200, 136), (128, 2048, 2048), (100, 1000, 8192)])
def test_linear_bfloat16(out_dtype, kind, M, N, K):
    if (kind == "skinny" and M > ops.WARP_LEVEL_MAX_ROWS) or (kind == "swapab" and M > ops.SKINNY_MAX_ROWS):
        pytest.skip("more rows than the weight-streaming kernels take")
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, seed=2)
    out = torch.empty(M, N, dtype=out_dtype, device=DEV)
    ops.linear(x, w, out, kind=kind)
    want = (x.double() @ w.double().T).float()
    if out_dtype == torch.bfloat16:
        torch.testing.assert_close(out.float(), want.to(torch.bfloat16).float(), rtol=1.6e-2, atol=1e-2 * math.sqrt(K / 64))
    else:
        torch.testing.assert_close(out, want, rtol=1e-4, atol=2e-3 * math.sqrt(K / 64))
    assert ops.bounded_wait_failures() == 0


@pytest.mark.parametrize("M,N,K", [(40, 38000, 136), (64, 19100, 520), (17, 300, 16384), (64, 2048, 2048), (33, 6144, 2048),
                                   (64, 2048, 8192), (20, 16384, 2048), (64, 130, 520), (50, 4096, 14336),
                                   (65, 6144, 2048), (128, 2048, 8192), (97, 391, 264), (120, 16384, 2048),
                                   (32, 6144, 2048), (24, 2048, 8192), (19, 16384, 2048), (32, 100, 64), (31, 4096, 14336),
                                   (48, 2048, 8192), (41, 16384, 2048), (80, 2048, 2048), (72, 16384, 2048), (66, 391, 520)])
def test_linear_swapab_slices_meet_in_a_cluster(M, N, K):
    """One CTA per (128-row tile, slice of k): more CTAs than the device holds at once
    (several waves), clusters of two, four and eight slices whose partial sums meet
    through distributed shared memory, a row tile that is not full, and the same
    bits on a second run (the slices are added in rank order)."""
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, seed=2)
    out = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.linear(x, w, out, kind="swapab")
    want = (x.double() @ w.double().T).float()
    torch.testing.assert_close(out, want, rtol=1e-4, atol=2e-3 * math.sqrt(K / 64))
    again = torch.full_like(out, float("nan"))
    ops.linear(x, w, again, kind="swapab")
    assert torch.equal(out, again)
    wide = torch.zeros(M, N + 24, dtype=torch.bfloat16, device=DEV)          # an output that is a column slice
    ops.linear(x, w, wide[:, 10:N + 10], kind="swapab")
    torch.testing.assert_close(wide[:, 10:N + 10].float(), want.to(torch.bfloat16).float(), rtol=1.6e-2, atol=1e-2 * math.sqrt(K / 64))
    assert float(wide[:, :10].abs().sum()) == 0 and float(wide[:, N + 10:].abs().sum()) == 0
    assert ops.bounded_wait_failures() == 0


def test_linear_strided_operands():
    """Inputs and outputs that are column slices of wider buffers."""
    xb, w = rnd(9, 304, dtype=torch.bfloat16), rnd(50, 96, dtype=torch.bfloat16, seed=3)
    x = xb[:, 8:104]
    outb = torch.zeros(9, 80, dtype=torch.bfloat16, device=DEV)
    ops.linear(x, w, outb[:, 10:60])
    want = (x.double() @ w.double().T).float().to(torch.bfloat16).float()
    torch.testing.assert_close(outb[:, 10:60].float(), want, rtol=1.6e-2, atol=1e-2)
    assert float(outb[:, :10].abs().sum()) == 0 and float(outb[:, 60:].abs().sum()) == 0


@pytest.mark.parametrize("M,N,K", [(1, 2048, 8192), (8, 2048, 2048), (3, 40, 14336), (16, 100, 20000),
                                   (2, 16, 32768 + 40), (4, 23700, 4096), (12, 9000, 6144), (2, 20000, 14336),
                                   (9, 4096, 14336), (5, 7000, 10240)])
def test_linear_skinny_long_rows_split_over_a_cluster(M, N, K):
    """Inner sizes beyond one pass: 2 to 8 CTAs share a row (their sums meet a batch
    of row tiles at a time: whole batches, a last short one, fewer tiles than ranks),
    and beyond that a CTA makes several passes."""
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, seed=2)
    out = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.linear(x, w, out, kind="skinny")
    want = (x.double() @ w.double().T).float()
    torch.testing.assert_close(out, want, rtol=1e-4, atol=2e-3 * math.sqrt(K / 64))
    again = torch.empty_like(out)
    ops.linear(x, w, again, kind="skinny")
    assert torch.equal(out, again)                    # fixed summation order
    assert ops.bounded_wait_failures() == 0


@pytest.mark.parametrize("kind", ["skinny", "swapab", "tcgen05"])
@pytest.mark.parametrize("M,I,K", [(1, 8, 96), (8, 264, 96), (16, 1000, 2048), (33, 24, 8192), (64, 264, 264),
                                   (200, 264, 96), (130, 1000, 2048), (96, 8192, 2048), (128, 264, 8192),
                                   (20, 8192, 2048), (32, 264, 96), (45, 8192, 2048), (80, 1000, 2048)])
def test_linear_with_fused_swiglu(kind, M, I, K):
    """The product over interleaved gate/up rows writes silu(gate) * up directly."""
    if (kind == "skinny" and M > ops.WARP_LEVEL_MAX_ROWS) or (kind == "swapab" and M > ops.SKINNY_MAX_ROWS):
        pytest.skip("more rows than the weight-streaming kernels take")
    x = rnd(M, K, dtype=torch.bfloat16, seed=1, scale=0.5)
    gate, up = rnd(I, K, dtype=torch.bfloat16, seed=2, scale=0.2), rnd(I, K, dtype=torch.bfloat16, seed=3, scale=0.2)
    w = ops.interleave_gate_up(gate, up)
    assert w.shape == (2 * I, K) and torch.equal(w[8:16], up[:8]) and torch.equal(w[16:24], gate[8:16]) if I >= 16 \
        else torch.equal(w[8:16], up[:8])
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.linear(x, w, out, kind=kind, epilogue="swiglu")
    g, u = x.double() @ gate.double().T, x.double() @ up.double().T
    want = (g / (1 + torch.exp(-g)) * u).float()
    torch.testing.assert_close(out.float(), want.to(torch.bfloat16).float(), rtol=2e-2, atol=2e-2 * math.sqrt(K / 64))
    assert ops.bounded_wait_failures() == 0


@pytest.mark.parametrize("M,N,K", [(129, 64, 64), (2048, 2048, 2048), (300, 144, 96), (130, 1000, 2056), (257, 2048, 8192),
                                   (192, 48, 64), (1000, 391, 264)])
def test_linear_adds_to_a_residual_stream(M, N, K):
    """residual += bfloat16(x . w^T) by tensor reductions in the product's epilogue:
    bit for bit what the product into a bfloat16 update, then the addition, give;
    row and column counts that are no multiples of the boxes; twice in a row."""
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, seed=2, scale=0.5)
    wide = rnd(M, N + 8, seed=3, scale=2.0)
    residual = wide[:, 4:N + 4] if N % 4 == 0 else rnd(M, N, seed=3, scale=2.0)   # a column slice where alignment allows
    before = residual.clone()
    plain = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops.linear(x, w, plain, kind="tcgen05")
    if not ops.linear_add_residual(x, w, residual):
        assert N % 4 != 0                                      # rows the tensor copies cannot address
        return
    assert torch.equal(residual, before + plain.float())
    assert ops.linear_add_residual(x, w, residual)
    assert torch.equal(residual, (before + plain.float()) + plain.float())
    if N % 4 == 0:
        assert torch.equal(wide[:, :4], rnd(M, N + 8, seed=3, scale=2.0)[:, :4])      # nothing beside the slice is touched
        assert torch.equal(wide[:, N + 4:], rnd(M, N + 8, seed=3, scale=2.0)[:, N + 4:])
    assert ops.bounded_wait_failures() == 0


def test_linear_does_not_add_to_a_residual_stream_what_it_cannot_serve():
    for M, N, K, dt in ((64, 64, 64, torch.bfloat16), (128, 64, 64, torch.bfloat16), (200, 64, 64, torch.float32),
                        (200, 64, 12, torch.bfloat16)):
        x, w = rnd(M, K, dtype=dt, seed=1), rnd(N, K, dtype=dt, seed=2)
        residual = rnd(M, N, seed=3)
        before = residual.clone()
        assert not ops.linear_add_residual(x, w, residual)
        assert torch.equal(residual, before)


def test_linear_refuses_unaligned_inner_size():
    x, w = rnd(4, 12, dtype=torch.bfloat16), rnd(5, 12, dtype=torch.bfloat16)
    with pytest.raises(ops.KernelError, match="multiples of 8"):
        ops.linear(x, w, torch.empty(4, 5, dtype=torch.bfloat16, device=DEV))


# ------------------------------------------------------------------- attention
def ref_attention(q, k, v, n_heads, n_kv, hd, pos_q, scale, window):
    """q [n, n_heads*hd] at positions pos_q over keys k, v [T, n_kv, hd] (float64)."""
    g = n_heads // n_kv
    kv_of_head = torch.arange(n_heads, device=q.device) // g
    out = torch.zeros(q.shape[0], n_heads, hd, dtype=torch.float64, device=q.device)
    qh = q.double().view(-1, n_heads, hd)
    for i, p in enumerate(pos_q):
        lo = max(0, p - window + 1) if window else 0
        kk = k[lo:p + 1].double()[:, kv_of_head]          # [keys, heads, hd]
        vv = v[lo:p + 1].double()[:, kv_of_head]
        w = torch.softmax(torch.einsum("thd,hd->ht", kk, qh[i]) * scale, dim=1)
        out[i] = torch.einsum("ht,thd->hd", w, vv)
    return out.view(q.shape[0], -1).float()


ATT_SHAPES = [(4, 2, 16), (3, 1, 48), (8, 8, 64), (6, 2, 128), (2, 1, 80), (20, 1, 32)]


def attention_case(dtype, n_heads, n_kv, hd, lens_before, lens_new, window, seed=0):
    """Sequences with `lens_before` tokens in the cache get `lens_new` more; returns
    what the kernels need and the reference output for the new tokens.  One far
    key of each sequence is made to dominate some queries."""
    cache = make_cache(n_kv, hd, dtype, n_pages=64)
    B = len(lens_before)
    slots = [cache.open_sequence() for _ in range(B)]
    if B > 1:                      # slots out of order
        slots = slots[::-1]
    scale = 1.0 / math.sqrt(hd)
    qs, wants, pos_all, tok_seq = [], [], [], []
    for b, (t0, n) in enumerate(zip(lens_before, lens_new)):
        T = t0 + n
        k = rnd(T, n_kv, hd, dtype=dtype, seed=seed + 10 * b + 1)
        v = rnd(T, n_kv, hd, dtype=dtype, seed=seed + 10 * b + 2)
        q = rnd(n, n_heads * hd, dtype=dtype, seed=seed + 10 * b + 3)
        far = min(3, T - 1)        # a key far from the end ...
        k[far] *= 4.0
        q[-1] = (k[far].float().repeat_interleave(n_heads // n_kv, dim=0).view(-1) * 1.5).to(dtype)
        fill_sequence(cache, 0, slots[b], k, v)
        pos = list(range(t0, T))
        wants.append(ref_attention(q, k, v, n_heads, n_kv, hd, pos, scale, window))
        qs.append(q)
        pos_all += pos
        tok_seq += [b] * n
    q = torch.cat(qs)
    want = torch.cat(wants)
    meta = dict(
        positions=torch.tensor(pos_all, dtype=torch.int32, device=DEV),
        token_seq=torch.tensor(tok_seq, dtype=torch.int32, device=DEV),
        slots=torch.tensor(slots, dtype=torch.int32, device=DEV),
        cu=torch.tensor(np.concatenate([[0], np.cumsum(lens_new)]), dtype=torch.int32, device=DEV),
        start=torch.tensor(lens_before, dtype=torch.int32, device=DEV),
    )
    return cache, q, want, meta, scale


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_heads,n_kv,hd", ATT_SHAPES + [(2, 2, 256)])
@pytest.mark.parametrize("window", [0, 37])
def test_attention_simple(dtype, n_heads, n_kv, hd, window):
    cache, q, want, m, scale = attention_case(dtype, n_heads, n_kv, hd, [0, 130, 63], [70, 1, 5], window)
    out = torch.empty_like(q)
    ops.attention_simple(q, out, cache.handles[0].kv, m["token_seq"], m["slots"], m["positions"],
                         n_heads, scale, window)
    torch.testing.assert_close(out.float(), want, **(dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32
                                                     else dict(rtol=2e-2, atol=2e-2)))


def test_attention_simple_on_the_reference_vector():
    """The reference's own attention case (model/attention_test.go:48-68: one query
    over 17 keys, 6 heads on 2, heads of 32, sin(0.013 i) inputs, scale 0.37) through
    the 32-bit attention kernel, against the float32 triple loop of that file, at its
    tolerance of 2e-5."""
    from test_plain import reference_attention_vector
    q, k, v, want, (T, n_heads, n_kv, hd, scale) = reference_attention_vector()
    cache = make_cache(n_kv, hd, torch.float32)
    slot = cache.open_sequence()
    fill_sequence(cache, 0, slot, torch.tensor(k, device=DEV).view(T, n_kv, hd), torch.tensor(v, device=DEV).view(T, n_kv, hd))
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    out = torch.empty(1, n_heads * hd, dtype=torch.float32, device=DEV)
    ops.attention_simple(torch.tensor(q, device=DEV).view(1, -1), out, cache.handles[0].kv, i32([0]), i32([slot]),
                         i32([T - 1]), n_heads, scale, 0)
    assert np.abs(out.cpu().numpy()[0] - want).max() < 2e-5


@pytest.mark.parametrize("n_heads,n_kv,hd", [(1, 1, 64), (6, 2, 64), (5, 5, 64), (8, 1, 64), (6, 2, 128), (3, 3, 128)])
@pytest.mark.parametrize("window", [0, 37, 64, 200])
@pytest.mark.parametrize("lens_before,lens_new", [([0], [1]), ([0, 0, 0], [5, 129, 64]), ([0], [128]),
                                                  ([10, 64, 100], [70, 1, 200]), ([0], [300]),
                                                  ([577, 0], [450, 1000])])
def test_attention_prefill_tcgen05(n_heads, n_kv, hd, window, lens_before, lens_new):
    cache, q, want, m, scale = attention_case(torch.bfloat16, n_heads, n_kv, hd, lens_before, lens_new, window)
    kv = cache.handles[0].kv
    assert ops.attention_tcgen05_supports(kv)
    qbuf = torch.zeros(q.shape[0], q.shape[1] + 16, dtype=torch.bfloat16, device=DEV)   # strided q
    qbuf[:, : q.shape[1]] = q
    out = torch.full_like(q, float("nan"))
    ops.attention_prefill_tcgen05(qbuf[:, : q.shape[1]], out, kv, m["cu"], m["slots"],
                                  m["start"], len(lens_new), max(lens_new), n_heads, scale, window)
    assert ops.bounded_wait_failures() == 0
    torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("n_heads,n_kv,hd", ATT_SHAPES)
@pytest.mark.parametrize("window", [0, 37, 64])
@pytest.mark.parametrize("lens_before,lens_new", [([0], [1]), ([0, 0, 0], [5, 129, 64]),
                                                  ([10, 64, 100], [70, 1, 200]), ([0], [300])])
def test_attention_prefill_bf16(n_heads, n_kv, hd, window, lens_before, lens_new):
    cache, q, want, m, scale = attention_case(torch.bfloat16, n_heads, n_kv, hd, lens_before, lens_new, window)
    qbuf = torch.zeros(q.shape[0], q.shape[1] + 16, dtype=torch.bfloat16, device=DEV)   # strided q
    qbuf[:, : q.shape[1]] = q
    out = torch.full_like(q, float("nan"))
    ops.attention_prefill_bf16(qbuf[:, : q.shape[1]], out, cache.handles[0].kv, m["cu"], m["slots"],
                               m["start"], len(lens_new), max(lens_new), n_heads, scale, window)
    torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("n_heads,n_kv,hd", ATT_SHAPES)
@pytest.mark.parametrize("window", [0, 37])
@pytest.mark.parametrize("splits", [1, 2, 5, 20])
def test_attention_decode_bf16(n_heads, n_kv, hd, window, splits):
    lens_before = [0, 63, 64, 700, 129]
    cache, q, want, m, scale = attention_case(torch.bfloat16, n_heads, n_kv, hd, lens_before,
                                              [1] * len(lens_before), window)
    out = torch.full_like(q, float("nan"))
    scratch = None
    if splits > 1:
        n = ops.attention_decode_scratch_floats(len(lens_before), n_heads, hd, splits)
        scratch = torch.full((n,), float("nan"), dtype=torch.float32, device=DEV)
    ops.attention_decode_bf16(q, out, cache.handles[0].kv, m["slots"], m["positions"], n_heads, scale,
                              window, splits, scratch)
    torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("n_heads,n_kv,hd", [(4, 2, 16), (8, 8, 64), (6, 2, 128)])
@pytest.mark.parametrize("window", [0, 100])
@pytest.mark.parametrize("splits,chunk", [(4, 3), (12, 1), (2, 4), (3, 2)])
def test_attention_decode_with_splits_sized_by_a_chunk_of_pages(n_heads, n_kv, hd, window, splits, chunk):
    """Sequences of very unequal lengths cut into parts of about `chunk` pages: short
    sequences leave splits without keys (the merge must pass over what those never
    wrote: the scratch is full of NaN), and a sequence longer than splits x chunk
    pages is cut into `splits` parts."""
    lens_before = [0, 63, 64, 700, 129, 450]
    cache, q, want, m, scale = attention_case(torch.bfloat16, n_heads, n_kv, hd, lens_before,
                                              [1] * len(lens_before), window)
    n = ops.attention_decode_scratch_floats(len(lens_before), n_heads, hd, splits)
    out = torch.full_like(q, float("nan"))
    scratch = torch.full((n,), float("nan"), dtype=torch.float32, device=DEV)
    ops.attention_decode_bf16(q, out, cache.handles[0].kv, m["slots"], m["positions"], n_heads, scale,
                              window, splits, scratch, chunk_pages=chunk)
    torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-2)
    deep = torch.full_like(q, float("nan"))               # the form with four pages in its ring: the same bits
    scratch.fill_(float("nan"))
    ops.attention_decode_bf16(q, deep, cache.handles[0].kv, m["slots"], m["positions"], n_heads, scale,
                              window, splits, scratch, chunk_pages=chunk, ring_pages=4)
    assert torch.equal(deep, out)


def test_the_decode_plan_follows_the_batch_not_the_data():
    """One long sequence alone is cut into many parts; many sequences are not cut at
    all; a batch of short sequences beside one long one gets a chunk that the short
    ones fit into whole; a window bounds the pages whatever the length."""
    one, chunk1, ring1 = ops.attention_decode_plan(1, 32, 32, 64, 8192, 0, 8192)
    assert one > 4 and (one - 1) * chunk1 < 128 <= one * chunk1 and ring1 == 3
    many, _, ring_many = ops.attention_decode_plan(64, 32, 32, 64, 2048, 0, 64 * 1100)
    assert many == 1 and ring_many == 3                   # 2,048 blocks fill the device without a cut
    mixed, chunk, _ = ops.attention_decode_plan(8, 32, 32, 64, 2048, 0, 8 * 1100)
    assert mixed >= 2 and chunk >= 8                      # a sequence of 500 tokens is one block
    windowed, wchunk, _ = ops.attention_decode_plan(1, 32, 32, 64, 100000, 256, 100000)
    assert windowed * wchunk <= 8                         # 256 keys touch five pages at most
    # about one block per place on the device, uncut: the form with the deeper ring (up to 64 channels only)
    assert ops.attention_decode_plan(16, 32, 32, 64, 2048, 0, 16 * 1100)[2] == 4
    assert ops.attention_decode_plan(16, 32, 8, 128, 2048, 0, 16 * 1100)[2] == 3
    with pytest.raises(ops.KernelError):
        ops.attention_decode_plan(1, 32, 5, 64, 100)


@pytest.mark.parametrize("n_heads,n_kv,hd", ATT_SHAPES + [(40, 2, 64)])
@pytest.mark.parametrize("window", [0, 37])
@pytest.mark.parametrize("splits", [1, 3, 16])
@pytest.mark.parametrize("rotate", [True, False])
def test_attention_decode_that_rotates_and_stores_the_new_token_itself(n_heads, n_kv, hd, window, splits, rotate):
    """Unrotated queries, keys and values of the new tokens as a projection leaves
    them: the kernel gives what rope_kv_store followed by the plain decode kernel
    gives, and leaves the same keys and values in the cache (new tokens at a page's
    first row, its last row, and in between)."""
    lens_before = [0, 63, 64, 700, 129]
    B = len(lens_before)
    q_dim, kv_dim = n_heads * hd, n_kv * hd
    caches, outs = [], []
    for fused in (False, True):
        cache = make_cache(n_kv, hd, torch.bfloat16, n_pages=64)
        slots = [cache.open_sequence() for _ in range(B)][::-1]
        for b, t0 in enumerate(lens_before):
            if t0:
                fill_sequence(cache, 0, slots[b], rnd(t0, n_kv, hd, dtype=torch.bfloat16, seed=10 * b + 1),
                              rnd(t0, n_kv, hd, dtype=torch.bfloat16, seed=10 * b + 2))
            cache.reserve(slots[b], t0 + 1)
        cache.flush_tables()
        kv = cache.handles[0].kv
        qkv = rnd(B, q_dim + 2 * kv_dim, dtype=torch.bfloat16, seed=77)
        slot_t = torch.tensor(slots, dtype=torch.int32, device=DEV)
        positions = torch.tensor(lens_before, dtype=torch.int32, device=DEV)
        token_seq = torch.arange(B, dtype=torch.int32, device=DEV)
        cos_sin = None
        if rotate:
            ang = rnd(B, hd // 2, seed=5, scale=3.0)
            cos_sin = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).contiguous()
        out = torch.full((B, q_dim), float("nan"), dtype=torch.bfloat16, device=DEV)
        n = ops.attention_decode_scratch_floats(B, n_heads, hd, splits)
        scratch = torch.full((max(n, 1),), float("nan"), dtype=torch.float32, device=DEV)
        if fused:
            ops.attention_decode_bf16(qkv[:, :q_dim], out, kv, slot_t, positions, n_heads, 0.2, window, splits, scratch,
                                      unrotated=(cos_sin, qkv[:, q_dim:q_dim + kv_dim], qkv[:, q_dim + kv_dim:], True))
        else:
            ops.rope_kv_store(qkv, cos_sin, n_heads, n_kv, hd, kv, token_seq, slot_t, positions)
            ops.attention_decode_bf16(qkv[:, :q_dim], out, kv, slot_t, positions, n_heads, 0.2, window, splits, scratch)
        outs.append(out.float())
        caches.append([read_sequence(cache, 0, slots[b], t0 + 1) for b, t0 in enumerate(lens_before)])
    assert torch.isfinite(outs[1]).all()
    torch.testing.assert_close(outs[1], outs[0], rtol=2e-2, atol=2e-2)
    for (k0, v0), (k1, v1) in zip(*caches):
        torch.testing.assert_close(k1.float(), k0.float(), rtol=1e-2, atol=1e-2)    # one rounding of the rotation
        assert torch.equal(v1, v0)


def test_attention_refuses_head_sizes_it_cannot_serve():
    assert not ops.attention_bf16_supports(40)
    assert not ops.attention_bf16_supports(144)
    assert ops.attention_bf16_supports(112)


# -------------------------------------------------------------------- sampling
@pytest.mark.parametrize("R,V", [(1, 5), (7, 391), (3, 49152), (2, 128257), (4, 128256), (5, 8192), (3, 50001)])
def test_argmax_first_maximum(R, V):
    logits = rnd(R, V + 3, seed=4)[:, :V] if V == 50001 else rnd(R, V, seed=4)   # 50001: rows 50004 apart
    logits[0, V - 1] = 50.0
    if R > 1:
        logits[1, 3] = 60.0
        logits[1, V // 2] = 60.0          # a tie: the lower index wins
    out = torch.zeros(R, dtype=torch.int32, device=DEV)
    ops.argmax(logits, out)
    want = [int(np.argmax(row)) for row in logits.cpu().numpy()]   # numpy: first maximum
    assert out.tolist() == want
    if R > 1:
        assert out[1].item() == 3


@pytest.mark.parametrize("R,V", [(64, 391), (6, 4096), (9, 49152), (5, 128256), (3, 128257), (4, 131073)])
def test_sample_temperature_matches_inverse_cdf(R, V):
    """Small rows take one block, rows up to 131072 entries a cluster of blocks that
    keep the row in shared memory, longer ones one block again."""
    import plain_llama
    T, seed = 0.8, 7
    logits = rnd(R, V, scale=2.0, seed=9)
    logits[0, V - 7] = 30.0                                  # one row whose mass sits in one late entry
    seq = torch.arange(R, dtype=torch.int32, device=DEV) % 5
    steps = torch.arange(R, dtype=torch.int32, device=DEV) // 5
    out = torch.zeros(R, dtype=torch.int32, device=DEV)
    ops.sample_temperature(logits, T, seed, seq, steps, out)
    lg = logits.cpu().numpy()
    for r in range(R):
        u = plain_llama.uniform(seed, int(seq[r]), int(steps[r]))
        cdf = np.cumsum(plain_llama.temperature_probs(lg[r], T))
        t = int(out[r])
        below = cdf[t - 1] if t > 0 else 0.0
        assert below - 1e-5 <= u <= cdf[t] + 1e-5, (r, t, u, below, cdf[t])
    # the same (seed, sequence, step) gives the same token whatever else is in the batch
    out2 = torch.zeros(1, dtype=torch.int32, device=DEV)
    k = R // 2
    ops.sample_temperature(logits[k:k + 1], T, seed, seq[k:k + 1].contiguous(), steps[k:k + 1].contiguous(), out2)
    assert out2.item() == out[k].item()
    assert out[0].item() == V - 7


def test_sample_temperature_follows_the_distribution():
    V, T = 50, 1.3
    logits = rnd(1, V, scale=1.5, seed=11).repeat(4000, 1).contiguous()
    seq = torch.zeros(4000, dtype=torch.int32, device=DEV)
    steps = torch.arange(4000, dtype=torch.int32, device=DEV)
    out = torch.zeros(4000, dtype=torch.int32, device=DEV)
    ops.sample_temperature(logits, T, 123, seq, steps, out)
    p = torch.softmax(logits[0].double() / T, 0).cpu().numpy()
    freq = np.bincount(out.cpu().numpy(), minlength=V) / 4000.0
    assert np.abs(freq - p).max() < 4 * np.sqrt(p.max() / 4000.0) + 1e-3
