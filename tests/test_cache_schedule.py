"""The cache's bookkeeping and the generation loop's decisions (no GPU)."""
import random

import pytest
import torch

import go_tinygrad_b200  # noqa: F401
from go_tinygrad_b200.cache import (Cache, CacheFull, CacheMisuse, KVRequest, PagePool, SlotTable,
                                    StateRequest)
from go_tinygrad_b200.engine.schedule import (RequestTooLarge, SequenceProgress, live,
                                              plan_batches)


def test_slot_table_never_loses_or_doubles_a_slot():
    table = SlotTable(5)
    rng = random.Random(0)
    held = set()
    for _ in range(2000):
        if held and (rng.random() < 0.5 or len(held) == 5):
            s = rng.choice(sorted(held))
            table.free(s)
            held.discard(s)
        else:
            s = table.alloc()
            assert s not in held and 0 <= s < 5
            held.add(s)
        assert set(table.held()) == held and table.n_free == 5 - len(held)
    for s in sorted(held):
        table.free(s)
    assert table.n_free == 5
    with pytest.raises(CacheMisuse, match="not held"):
        table.free(0)
    with pytest.raises(CacheMisuse):
        table.free(7)
    got = [table.alloc() for _ in range(5)]
    assert sorted(got) == [0, 1, 2, 3, 4]
    with pytest.raises(CacheFull):
        table.alloc()


def test_page_pool_accounts_for_every_page():
    pool = PagePool(6)
    a = pool.alloc(2, slot=0)
    b = pool.alloc(3, slot=1)
    assert len(set(a) | set(b)) == 5 and pool.n_free == 1
    with pytest.raises(CacheFull):
        pool.alloc(2, slot=2)
    assert pool.n_free == 1                               # a refused request takes nothing
    with pytest.raises(CacheMisuse, match="belongs to"):
        pool.free(a, slot=1)
    pool.free(a, slot=0)
    with pytest.raises(CacheMisuse):
        pool.free(a, slot=0)                              # freed twice
    assert pool.owned_by(1) == sorted(b) and pool.n_free == 3


def make_cache(max_tokens=64 * 6, max_slots=3):
    requests = [[KVRequest(2, 16)], [KVRequest(2, 16)], [KVRequest(1, 32, window=128)],
                [StateRequest("h", (4,))], []]
    return Cache(requests, [None, None, None, None, 1], max_tokens=max_tokens, max_slots=max_slots,
                 dtype=torch.float32, device="cpu")


def test_groups_have_storage_of_their_own():
    cache = make_cache()
    assert len(cache.groups) == 2                         # all-keys layers and the windowed layer
    full, win = cache.groups
    assert full.storage.shape == (2, 6, 2, 2, 64, 16) and win.storage.shape == (1, 6, 2, 1, 64, 32)
    assert cache.handles[0].kv.k.data_ptr() != cache.handles[1].kv.k.data_ptr()
    assert cache.handles[2].kv.window == 128 and cache.handles[0].kv.window is None
    assert cache.handles[3].kv is None and cache.handles[3].state("h").shape == (3, 4)
    shared = cache.handles[4]                             # reads entry 1's keys, writes none
    assert not shared.writes and shared.kv.k.data_ptr() == cache.handles[1].kv.k.data_ptr()
    assert cache.handles[1].writes


def test_sequences_take_and_return_pages():
    cache = make_cache()
    a, b = cache.open_sequence(), cache.open_sequence()
    cache.reserve(a, 65)
    cache.reserve(b, 64)
    assert cache.free_pages() == [3, 3] and cache.tokens_held() == 192
    cache.advance(a, 65)
    cache.advance(b, 10)
    assert (cache.length(a), cache.length(b)) == (65, 10)
    with pytest.raises(CacheMisuse, match="without reserved pages"):
        cache.advance(b, 60)
    # block tables: the pages a sequence got, in order, distinct across sequences and groups' own
    for grp in cache.groups:
        pa, pb = grp.pages_of[a], grp.pages_of[b]
        assert grp.table_host[a, :2].tolist() == pa and grp.table_host[b, :1].tolist() == pb
        assert not set(pa) & set(pb)
    with pytest.raises(CacheFull, match="full"):
        cache.reserve_many([(a, 65 + 128), (b, 64 + 128)])
    assert cache.free_pages() == [3, 3]                   # all or nothing
    # this cache holds a record of fixed size too: a shorter length would leave the
    # record as it is, so rolling back is refused rather than silently wrong
    with pytest.raises(CacheMisuse, match="fixed size"):
        cache.truncate(a, 3)
    assert cache.length(a) == 65
    cache.close_sequence(a)
    assert cache.free_pages() == [5, 5] and cache.open_slots() == [b]
    with pytest.raises(CacheMisuse, match="not open"):
        cache.close_sequence(a)
    with pytest.raises(CacheMisuse):
        cache.reserve(a, 1)
    cache.close_sequence(b)
    assert cache.free_pages() == [6, 6] and cache.open_slots() == [] and cache.tokens_held() == 0


def test_truncate_forgets_tokens_of_a_cache_of_keys_and_values():
    cache = Cache([[KVRequest(2, 16)], [KVRequest(1, 32, window=128)]], [None, None], max_tokens=64 * 4,
                  max_slots=2, dtype=torch.float32, device="cpu")
    a = cache.open_sequence()
    cache.reserve(a, 65)
    cache.advance(a, 65)
    cache.truncate(a, 3)
    assert cache.length(a) == 3 and cache.free_pages() == [2, 2]      # the pages stay with the sequence
    with pytest.raises(CacheMisuse):
        cache.truncate(a, 4)
    cache.close_sequence(a)
    assert cache.free_pages() == [4, 4]


def test_the_longest_sequence_is_counted_in_tokens_not_pages():
    # a model whose longest position is no multiple of the page size: positions up to
    # 99 exist, position 100 does not, although its page is there
    cache = Cache([[KVRequest(2, 16)]], [None], max_tokens=64 * 8, max_slots=2, max_position=100,
                  dtype=torch.float32, device="cpu")
    assert cache.max_sequence == 100 and cache.pages_per_seq == 2
    a, b = cache.open_sequence(), cache.open_sequence()
    cache.reserve(a, 100)
    with pytest.raises(CacheFull, match="longest"):
        cache.reserve(a, 101)
    with pytest.raises(CacheFull, match="longest"):
        cache.reserve_many([(b, 64), (a, 101)])
    assert cache.free_pages() == [6]                      # the refused step took nothing for b either
    cache.reserve_many([(b, 64), (a, 100)])
    assert cache.free_pages() == [5]


def test_slots_are_used_again_and_state_starts_at_zero():
    cache = make_cache()
    seen = set()
    for round_ in range(4):
        slots = [cache.open_sequence() for _ in range(3)]
        with pytest.raises(CacheFull, match="slots"):
            cache.open_sequence()
        for s in slots:
            assert float(cache.handles[3].state("h")[s].abs().sum()) == 0.0
            cache.handles[3].state("h")[s] += 1.0 + round_     # a mixer leaves state behind
            cache.reserve(s, 100)
            cache.advance(s, 100)
            seen.add(s)
        for s in slots:
            cache.close_sequence(s)
    assert seen == {0, 1, 2} and cache.free_pages() == [6, 6]


def test_a_sequence_cannot_outgrow_the_table():
    cache = Cache([[KVRequest(1, 16)]], [None], max_tokens=64 * 10, max_slots=2, max_position=200,
                  dtype=torch.float32, device="cpu")
    assert cache.pages_per_seq == 4 and cache.max_sequence == 200
    s = cache.open_sequence()
    cache.reserve(s, 200)
    with pytest.raises(CacheFull, match="longest"):
        cache.reserve(s, 201)
    # without a model's limit the table's pages decide
    cache = Cache([[KVRequest(1, 16)]], [None], max_tokens=64 * 4, max_slots=2, dtype=torch.float32, device="cpu")
    s = cache.open_sequence()
    cache.reserve(s, 256)
    with pytest.raises(CacheFull, match="longest"):
        cache.reserve(s, 257)


# ----------------------------------------------------------------- the loop's decisions
def test_batches_fit_the_cache_and_keep_order():
    lengths = [5, 70, 17, 1, 64, 130, 3]
    new = [9, 3, 20, 12, 1, 6, 33]
    batches = plan_batches(lengths, new, max_tokens=64 * 5, max_batch=4)
    assert [i for b in batches for i in b] == list(range(7))
    for b in batches:
        assert len(b) <= 4
        assert sum((lengths[i] + new[i] - 1 + 63) // 64 * 64 for i in b) <= 64 * 5
    assert plan_batches([10, 10, 10], [5, 5, 5], max_tokens=64 * 8, max_batch=2) == [[0, 1], [2]]
    assert plan_batches([64], [1], max_tokens=64, max_batch=1) == [[0]]      # the last token is not fed back
    with pytest.raises(RequestTooLarge, match="cache holds"):
        plan_batches([100], [100], max_tokens=128, max_batch=4)
    with pytest.raises(RequestTooLarge, match="longest"):
        plan_batches([300], [1], max_tokens=1024, max_batch=4, max_sequence=256)
    assert plan_batches([250], [100], max_tokens=256, max_batch=4, max_sequence=256) == [[0]]
    with pytest.raises(ValueError, match="empty"):
        plan_batches([0], [1], max_tokens=64, max_batch=1)


def test_a_sequence_ends_on_stop_length_or_capacity():
    s = SequenceProgress(0, prompt_length=4, max_new_tokens=3, stop={9})
    s.start()
    s.accept(5)
    assert not s.finished
    s.accept(9)
    assert s.finish_reason == "stop" and s.tokens == [5, 9]      # the stop token is kept
    with pytest.raises(RuntimeError):
        s.accept(1)
    t = SequenceProgress(1, 4, 2, {9})
    t.start(); t.accept(1); t.accept(2)
    assert t.finish_reason == "length"
    z = SequenceProgress(2, 4, 0, set())
    z.start()
    assert z.finished and z.tokens == []
    c = SequenceProgress(3, prompt_length=6, max_new_tokens=10, stop=set(), max_sequence=8)
    c.start(); c.accept(1); c.accept(2)
    assert not c.finished                                   # 8 tokens fit positions 0..7
    c.accept(3)
    assert c.finish_reason == "capacity" and len(c.tokens) == 3
    assert live([s, t, z, c, SequenceProgress(4, 1, 1, set())])[0].request == 4


def test_a_group_that_keeps_a_window_gives_back_the_pages_that_slid_out_of_it():
    """Two groups: all keys, and a window of 100.  As the sequence grows the windowed
    group holds only the pages its next token can still see; the other keeps all.  No
    page is lost, held twice or freed twice, and a released page serves another sequence."""
    cache = Cache([[KVRequest(2, 16)], [KVRequest(1, 32, window=100)]], [None, None], max_tokens=64 * 12,
                  max_slots=2, dtype=torch.float32, device="cpu")
    full, win = cache.groups
    a = cache.open_sequence()
    cache.reserve(a, 300)                                  # a prompt: every page is needed while it runs
    assert cache.free_pages() == [7, 7]
    first = list(win.pages_of[a])
    cache.advance(a, 300)
    # the next token, at position 300, sees keys 201..300: pages 3 and 4; 0..2 went back
    assert cache.free_pages() == [7, 10]
    assert win.pages_of[a] == [-1, -1, -1] + first[3:] and full.pages_of[a] == full.table_host[a, :5].tolist()
    assert cache.tokens_held() == 5 * 64
    for length in range(301, 400):                         # one token at a time
        cache.reserve(a, length)
        cache.advance(a, 1)
        lo = (length - 100 + 1) // 64
        held = [i for i, p in enumerate(win.pages_of[a]) if p >= 0]
        assert held == list(range(lo, (length - 1) // 64 + 1)), length
        assert win.pool.n_free == 12 - len(held) and full.pool.n_free == 12 - ((length + 63) // 64)
    # a page that was given back goes to another sequence, and is not this one's any more
    b = cache.open_sequence()
    cache.reserve(b, 64 * 5)
    assert not set(p for p in win.pages_of[a] if p >= 0) & set(win.pages_of[b])
    assert set(first[:3]) <= set(win.pages_of[b]) | set(win.pages_of[a])      # in use again, by b or by a itself
    assert set(first[:3]) & set(win.pages_of[b])
    # going back: within what is still held it works, below it is refused
    cache.truncate(a, 390)
    with pytest.raises(CacheMisuse, match="given back"):
        cache.truncate(a, 200)
    assert cache.length(a) == 390
    cache.close_sequence(a)
    cache.close_sequence(b)
    assert cache.free_pages() == [12, 12] and cache.tokens_held() == 0
    assert sorted(win.pool.alloc(12, 0)) == list(range(12))  # every page once


def test_the_workspace_hands_out_nothing_twice_before_it_is_told_to():
    """Scratch of a step: a region for the whole step and two that take turns layer by
    layer.  A tensor stays untouched until the layer after its own has ended; regions
    start empty, serve ordinary tensors meanwhile, and grow at the next reset; without
    the engine's calls nothing is ever reused."""
    from go_tinygrad_b200.parts.base import Runtime, Workspace
    rt = Runtime(torch.device("cpu"), torch.float32)
    ws = rt.workspace
    assert isinstance(ws, Workspace) and ws.buffers() == []

    def one_step(check_reuse):
        ws.begin_step()
        residual = rt.empty(4, 8, lifetime="step")
        residual.fill_(7.0)
        kept = []
        for layer in range(5):
            ws.next_layer()
            a, b = rt.empty(3, 5), rt.empty(100, dtype=torch.int32)
            assert a.dtype == torch.float32 and b.dtype == torch.int32 and a.shape == (3, 5)
            assert a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0      # on the device: 256, from an aligned buffer
            a.fill_(float(layer))
            b.fill_(layer)
            kept.append((a, b))
            if layer:                                      # the layer before is still whole
                assert float(kept[layer - 1][0].min()) == float(layer - 1) and int(kept[layer - 1][1].max()) == layer - 1
            if check_reuse and layer >= 2:                 # the one before that has been handed out again
                assert kept[layer - 2][0].data_ptr() == a.data_ptr()
        assert float(residual.min()) == 7.0
        return residual, kept
    first, kept = one_step(check_reuse=False)              # nothing to cut from at first: ordinary tensors, and
    assert len({t.data_ptr() for pair in kept[:2] for t in pair}) == 4      # the layers' regions appear as they take turns
    ws.begin_step()                                        # now the regions exist, as large as was asked for
    assert len(ws.buffers()) == 3
    held = [b.data_ptr() for b in ws.buffers()]
    second, _ = one_step(check_reuse=True)
    third, _ = one_step(check_reuse=True)
    assert second.data_ptr() == third.data_ptr() and [b.data_ptr() for b in ws.buffers()] == held   # the same memory, no growth
    # a larger step: served, and the regions have grown by the step after it
    ws.begin_step()
    big = rt.empty(1000, 1000, lifetime="step")
    big.zero_()
    assert [b.data_ptr() for b in ws.buffers()] == held
    ws.begin_step()
    assert ws.step_region.buffer.numel() >= 4 * 1000 * 1000
    with pytest.raises(ValueError):
        rt.empty(3, lifetime="forever")
    # without the engine's calls nothing is reused
    rt2 = Runtime(torch.device("cpu"), torch.bfloat16)
    alive = [rt2.empty(16, 16) for _ in range(50)]
    assert len({t.data_ptr() for t in alive}) == 50 and rt2.empty(2, 2).dtype == torch.bfloat16
    assert rt2.result(3, 3).shape == (3, 3)
