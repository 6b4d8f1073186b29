"""The schedules the measurement runs, checked for what they compute: decode
attention over 8,192 keys per sequence at the split counts the library picks for
1, 8 and 64 sequences; prompt attention and the projection that rotates and stores
in its epilogue at 2,048 and 8,192 tokens; decode steps of 17, 33 and 64 sequences
through the engine at the layer shapes of the three models (the tensor-core product
with swapped operands, whose slices of k meet in a cluster, and its fused SwiGLU);
and a decode batch
replayed as a CUDA graph against the same steps launched in the open."""
import math

import numpy as np
import pytest
import torch

import go_tinygrad_b200 as lib
import plain_llama
from go_tinygrad_b200.cache import Cache, KVRequest
from go_tinygrad_b200.engine import StepEntry, step
from go_tinygrad_b200.engine.decode import DecodeBatch
from go_tinygrad_b200.kernels import ops
from test_real_shapes_gpu import SHAPES, check

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF16 = torch.bfloat16


def gpu_rnd(*shape, seed, scale=1.0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(*shape, generator=g, device=DEV) * scale).to(BF16)


def scattered_cache(n_kv, hd, n_seqs, pages_per_seq, seed=5):
    """One cache entry whose pages are handed out in a scrambled order."""
    n_pages = n_seqs * pages_per_seq
    cache = Cache([[KVRequest(n_kv, hd)]], [None], max_tokens=n_pages * 64, max_slots=n_seqs, dtype=BF16, device=DEV)
    cache.groups[0].pool._free = [int(p) for p in np.random.default_rng(seed).permutation(n_pages)]
    return cache


def put(cache, slot, k, v):
    """k, v [T, n_kv, hd] become the first T tokens of `slot`."""
    T = k.shape[0]
    cache.reserve(slot, T)
    kv = cache.handles[0].kv
    t = torch.arange(T)
    pages = cache.groups[0].table_host[slot][t // 64].long().to(DEV)
    kv.k[pages, :, (t % 64).to(DEV), :] = k
    kv.v[pages, :, (t % 64).to(DEV), :] = v
    cache._length[slot] = T


def decode_reference(q, k, v, n_heads, n_kv, scale):
    """One query [n_heads*hd] over keys and values [T, n_kv, hd], float64."""
    hd = k.shape[-1]
    qh = q.double().view(n_kv, n_heads // n_kv, hd)
    s = torch.einsum("tkd,kgd->kgt", k.double(), qh) * scale
    w = torch.softmax(s, dim=-1)
    return torch.einsum("kgt,tkd->kgd", w, v.double()).reshape(-1).float()


# ----------------------------------------------------- decode attention, 8,192 keys
def lens_for(n_seqs):
    """Tokens already in the cache: the new token at a page's last row, its first row, in between."""
    return [8191, 8128, 8127, 8000][:n_seqs] + [int(x) for x in np.random.default_rng(1).integers(7000, 8192, max(0, n_seqs - 4))]


@pytest.mark.parametrize("rotate_and_store", [False, True])
@pytest.mark.parametrize("n_seqs", [1, 8, 64])
@pytest.mark.parametrize("model_heads,n_heads,n_kv,hd", [((32, 32), 8, 8, 64), ((32, 8), 16, 4, 128)])
def test_decode_attention_over_8192_keys(model_heads, n_heads, n_kv, hd, n_seqs, rotate_and_store):
    """128 pages per sequence, the ring of three (or four) pages wrapping dozens of
    times, at the split count the library chooses for this many sequences of the
    model's head counts (the test itself runs fewer heads so that 64 sequences of
    8,192 keys stay small).  In every sequence one key far from the end and one in
    the middle are made to dominate some heads' queries; the new token sits at a
    page's last row, its first row, or in between."""
    splits, chunk, ring = ops.attention_decode_plan(n_seqs, model_heads[0], model_heads[1], hd, 8192, 0, sum(lens_for(n_seqs)) + n_seqs)
    assert 1 <= splits <= 64 and (splits - 1) * chunk < 128 <= splits * chunk
    if n_seqs == 1:
        assert splits > 4            # one sequence alone has to be cut to fill the device
    cache = scattered_cache(n_kv, hd, n_seqs, 128)
    scale = 1.0 / math.sqrt(hd)
    lens = lens_for(n_seqs)
    slots = [cache.open_sequence() for _ in range(n_seqs)][::-1]
    group = n_heads // n_kv
    qs, wants, new_kv = [], [], []
    for b, t0 in enumerate(lens):
        T = t0 + 1
        k, v = gpu_rnd(T, n_kv, hd, seed=10 * b + 1), gpu_rnd(T, n_kv, hd, seed=10 * b + 2)
        q = gpu_rnd(n_heads, hd, seed=10 * b + 3)
        far, mid = 3 + b % 50, T // 2 + b
        k[far] *= 3.0
        k[mid] *= 3.0
        q[0] = k[far, 0] * 1.5                                  # the first head looks at the far key
        q[n_heads - 1] = k[mid, n_kv - 1] * 1.5                 # the last head at the one in the middle
        wants.append(decode_reference(q.reshape(-1), k, v, n_heads, n_kv, scale))
        put(cache, slots[b], k[:t0] if rotate_and_store else k, v[:t0] if rotate_and_store else v)
        if rotate_and_store:
            cache.reserve(slots[b], T)
        qs.append(q.reshape(-1))
        new_kv.append((k[t0].reshape(-1), v[t0].reshape(-1)))
    cache.flush_tables()
    kv = cache.handles[0].kv
    slot_t = torch.tensor(slots, dtype=torch.int32, device=DEV)
    positions = torch.tensor(lens, dtype=torch.int32, device=DEV)
    out = torch.full((n_seqs, n_heads * hd), float("nan"), dtype=BF16, device=DEV)
    n = ops.attention_decode_scratch_floats(n_seqs, n_heads, hd, splits)
    scratch = torch.full((max(n, 1),), float("nan"), dtype=torch.float32, device=DEV)
    if rotate_and_store:
        # the projection's row as the kernel finds it in a decode step: q | k | v, unrotated
        # (no rotation table: the keys above are what the cache should hold as they are)
        qkv = torch.cat([torch.stack(qs), torch.stack([a for a, _ in new_kv]), torch.stack([b for _, b in new_kv])], dim=1)
        qd, kd = n_heads * hd, n_kv * hd
        ops.attention_decode_bf16(qkv[:, :qd], out, kv, slot_t, positions, n_heads, scale, 0, splits, scratch,
                                  unrotated=(None, qkv[:, qd:qd + kd], qkv[:, qd + kd:], True), chunk_pages=chunk,
                                  ring_pages=ring)
        for b, t0 in enumerate(lens):                           # and the new token is in the cache afterwards
            page = int(cache.groups[0].table_host[slots[b]][t0 // 64])
            assert torch.equal(kv.k[page, :, t0 % 64, :].reshape(-1), new_kv[b][0])
            assert torch.equal(kv.v[page, :, t0 % 64, :].reshape(-1), new_kv[b][1])
    else:
        ops.attention_decode_bf16(torch.stack(qs), out, kv, slot_t, positions, n_heads, scale, 0, splits, scratch,
                                  chunk_pages=chunk, ring_pages=ring)
    torch.testing.assert_close(out.float(), torch.stack(wants), rtol=2e-2, atol=2e-2)
    # the engineered heads really saw their key: their output is that key's value, nearly
    for b in (0, n_seqs - 1):
        page = int(cache.groups[0].table_host[slots[b]][(3 + b % 50) // 64])
        v_far = kv.v[page, 0, (3 + b % 50) % 64, :].float()
        assert (out[b, :hd].float() - v_far).abs().max() < 0.15 * v_far.abs().max()


# ----------------------------------------------------- prompt attention, 2,048 and 8,192 tokens
def prompt_reference(q, k, v, n_heads, n_kv, start, scale):
    """Causal attention of queries at positions start.. over keys 0.., float64, head by head."""
    n, hd = q.shape[0], k.shape[-1]
    T = k.shape[0]
    out = torch.empty(n, n_heads, hd, dtype=torch.float32, device=q.device)
    qh = q.view(n, n_heads, hd)
    allowed = torch.arange(T, device=q.device)[None, :] <= (start + torch.arange(n, device=q.device))[:, None]
    for h in range(n_heads):
        kvh = h // (n_heads // n_kv)
        s = (qh[:, h].double() @ k[:, kvh].double().T) * scale
        s.masked_fill_(~allowed, float("-inf"))
        out[:, h] = (torch.softmax(s, dim=1) @ v[:, kvh].double()).float()
    return out.view(n, -1)


@pytest.mark.parametrize("before,new", [(0, 2048), (0, 8192), (4096, 4096), (8191 - 300, 301)])
@pytest.mark.parametrize("n_heads,n_kv,hd", [(4, 4, 64), (4, 1, 128)])
def test_prompt_attention_at_2048_and_8192_tokens(n_heads, n_kv, hd, before, new):
    """Whole prompts of the measured lengths, the second half of an 8,192-token
    prompt over its first half, and a tail that ends at the last position.  The last
    query is made to look at a key in the first page, the one in the middle at its own
    neighbour."""
    T = before + new
    cache = scattered_cache(n_kv, hd, 1, (T + 63) // 64)
    slot = cache.open_sequence()
    scale = 1.0 / math.sqrt(hd)
    k, v = gpu_rnd(T, n_kv, hd, seed=1), gpu_rnd(T, n_kv, hd, seed=2)
    q = gpu_rnd(new, n_heads, hd, seed=3)
    k[5] *= 3.0
    q[-1] = (k[5] * 1.5).repeat_interleave(n_heads // n_kv, dim=0)
    k[before + new // 2 - 1] *= 3.0
    q[new // 2] = (k[before + new // 2 - 1] * 1.5).repeat_interleave(n_heads // n_kv, dim=0)
    q = q.reshape(new, -1)
    put(cache, slot, k, v)
    cache.flush_tables()
    kv = cache.handles[0].kv
    assert ops.attention_tcgen05_supports(kv)
    want = prompt_reference(q, k, v, n_heads, n_kv, before, scale)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    out = torch.full_like(q, float("nan"))
    ops.attention_prefill_tcgen05(q, out, kv, i32([0, new]), i32([slot]), i32([before]), 1, new, n_heads, scale, 0)
    assert ops.bounded_wait_failures() == 0
    torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-2)
    out2 = torch.full_like(q, float("nan"))              # the warp-level kernel takes the same case
    ops.attention_prefill_bf16(q, out2, kv, i32([0, new]), i32([slot]), i32([before]), 1, new, n_heads, scale, 0)
    torch.testing.assert_close(out2.float(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("M", [2048, 8192])
def test_projection_with_rotation_and_cache_store_at_2048_and_8192_tokens(M):
    """The query/key/value product of a whole prompt at the measured width (32
    heads of 64 channels on a width of 2,048): rotated queries out, rotated keys and
    values in the cache, against a float64 product and rotation."""
    n_heads = n_kv = 32
    hd, K = 64, 2048
    cache = scattered_cache(n_kv, hd, 2, M // 64)
    cache.open_sequence()
    slot = cache.open_sequence()
    cache.reserve(slot, M)
    cache.flush_tables()
    width = (n_heads + 2 * n_kv) * hd
    x, w = gpu_rnd(M, K, seed=3, scale=0.5), gpu_rnd(width, K, seed=4, scale=0.05)
    positions = torch.arange(M, dtype=torch.int32, device=DEV)
    token_seq = torch.zeros(M, dtype=torch.int32, device=DEV)
    slot_t = torch.tensor([slot], dtype=torch.int32, device=DEV)
    inv = torch.tensor([1.0 / math.pow(130000.0, 2 * i / hd) for i in range(32)], dtype=torch.float64, device=DEV)
    cs = torch.empty(M, 32, 2, dtype=torch.float32, device=DEV)
    ops.rope_table(positions, inv, cs)
    kv = cache.handles[0].kv
    qkv = torch.full((M, width), 7.0, dtype=BF16, device=DEV)
    assert ops.qkv_rope_fused_supports(x, w, qkv, cs, n_heads, n_kv, hd, kv)
    ops.linear_qkv_rope(x, w, qkv, cs, n_heads, n_kv, kv, token_seq, slot_t, positions)
    assert ops.bounded_wait_failures() == 0
    close = dict(rtol=1.6e-2, atol=2e-2)
    c, s = cs[:, None, :, 0].double(), cs[:, None, :, 1].double()
    t = torch.arange(M)
    pages = cache.groups[0].table_host[slot][t // 64].long().to(DEV)
    for lo in range(0, M, 2048):                          # in row blocks, to keep the float64 product small
        rows = slice(lo, lo + 2048)
        full = x[rows].double() @ w.double().T

        def rot(part, nh):
            part = part.reshape(-1, nh, hd)
            a, b = part[..., :32], part[..., 32:]
            return torch.cat([a * c[rows] - b * s[rows], a * s[rows] + b * c[rows]], dim=-1)
        torch.testing.assert_close(qkv[rows, : n_heads * hd].float(), rot(full[:, : n_heads * hd], n_heads).reshape(2048, -1).float(), **close)
        got_k = kv.k[pages[rows], :, (t[rows] % 64).to(DEV), :]
        got_v = kv.v[pages[rows], :, (t[rows] % 64).to(DEV), :]
        torch.testing.assert_close(got_k.float(), rot(full[:, n_heads * hd: (n_heads + n_kv) * hd], n_kv).float(), **close)
        torch.testing.assert_close(got_v.float(), full[:, (n_heads + n_kv) * hd:].reshape(-1, n_kv, hd).float(), **close)
    assert float((qkv[:, n_heads * hd:].float() - 7.0).abs().sum()) == 0.0


# ----------------------------------------------------- decode steps of 17, 33 and 64 sequences
@pytest.fixture(scope="module", params=list(SHAPES))
def peaked(request, tmp_path_factory):
    """A one- or two-layer model at a real layer shape whose weights are twice as
    large as a trained model's, so that attention is peaked and logits are large:
    a wrong key, row or page moves them by far more than the tolerance."""
    name = request.param
    folder = str(tmp_path_factory.mktemp(f"peaked_{name}"))
    lib.write_random_model(folder, SHAPES[name], seed=21, dtype="bfloat16", std=0.04, norm_std=0.05)
    return name, folder, plain_llama.read_model(folder)


@pytest.mark.parametrize("n_seqs", [17, 33, 64])
def test_decode_steps_of_17_to_64_sequences(peaked, n_seqs):
    """Prompts of unequal lengths together, then three tokens each: the decode steps
    take the products for 17 to 64 rows.  Every sequence is compared."""
    name, folder, (cfg, w) = peaked
    rng = np.random.default_rng(n_seqs)
    decoded = 3
    lengths = rng.integers(2, 12, n_seqs).tolist()
    lengths[0], lengths[-1] = 70, 1                      # one that crosses a page, one of a single token
    requests = [rng.integers(0, cfg["vocab_size"], n + decoded).tolist() for n in lengths]
    want = [plain_llama.forward(cfg, w, r) for r in requests]
    model = lib.Model.load(folder, dtype="bfloat16", device="cuda")
    cache = model.new_cache(max_tokens=64 * (n_seqs + 1), max_slots=n_seqs)
    slots = [cache.open_sequence() for _ in requests]
    got = step(model, cache, [StepEntry(s, r[:n], [n - 1]) for s, r, n in zip(slots, requests, lengths)])
    got = got.float().cpu().numpy()
    widest = cfg["intermediate_size"]
    for i, n in enumerate(lengths):
        check(got[i], want[i][n - 1], "bfloat16", widest, f"{name}: last prompt token of sequence {i} of {n_seqs}")
    for t in range(decoded):
        logits = step(model, cache, [StepEntry(s, [r[n + t]], [0]) for s, r, n in zip(slots, requests, lengths)])
        logits = logits.float().cpu().numpy()
        for i, n in enumerate(lengths):
            check(logits[i], want[i][n + t], "bfloat16", widest, f"{name}: decoded token {t} of sequence {i} of {n_seqs}")
    assert ops.bounded_wait_failures() == 0


@pytest.mark.parametrize("n_seqs", [3, 24])
def test_a_replayed_decode_batch_gives_what_the_open_steps_give(peaked, n_seqs):
    """The decode step recorded as a CUDA graph and replayed, against the same steps
    launched kernel by kernel: the same tokens, the same logits to rounding (the two
    may split a sequence's keys differently), and both equal to the plain
    implementation fed the same tokens."""
    name, folder, (cfg, w) = peaked
    rng = np.random.default_rng(100 + n_seqs)
    lengths = rng.integers(3, 40, n_seqs).tolist()
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in lengths]
    model = lib.Model.load(folder, dtype="bfloat16", device="cuda")
    n_steps = 6
    runs = {}
    for use_graph in (False, True):
        cache = model.new_cache(max_tokens=64 * 2 * n_seqs, max_slots=n_seqs)
        slots = [cache.open_sequence() for _ in prompts]
        logits = step(model, cache, [StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        tokens = logits.argmax(dim=1).tolist()
        batch = DecodeBatch(model, cache, slots, list(range(n_seqs)), lib.Sampler(0.0, 0), use_graph=use_graph)
        fed, seen = [tokens], []
        for i in range(n_steps):
            tokens = batch.step_host(tokens, [i + 1] * n_seqs)
            seen.append(batch.logits.float().cpu().numpy().copy())
            fed.append(tokens)
        assert (batch.graph is not None) == use_graph
        runs[use_graph] = (fed, seen)
    assert runs[True][0] == runs[False][0], "the replayed batch sampled other tokens"
    for a, b in zip(runs[True][1], runs[False][1]):
        assert np.abs(a - b).max() <= 1e-2 * max(1.0, np.abs(b).max())
    fed, seen = runs[True]
    for i in (0, n_seqs // 2, n_seqs - 1):
        seq = prompts[i] + [fed[t][i] for t in range(n_steps)]
        want = plain_llama.forward(cfg, w, seq)
        for t in range(n_steps):
            check(seen[t][i], want[len(prompts[i]) + t], "bfloat16", cfg["intermediate_size"],
                  f"{name}: replayed step {t} of sequence {i}")
