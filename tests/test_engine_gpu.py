"""The engine against the plain implementation, in float32 and in bfloat16, under
every way of cutting the same requests: whole, the last 32 tokens one by one,
in batches of unequal lengths whose shorter requests end earlier, one batch
after another so that slots and pages are used again, long decoding, and the
first tokens of a sequence."""
import numpy as np
import pytest
import torch

import go_tinygrad_b200  # noqa: F401
from go_tinygrad_b200.engine import Model, StepEntry, StepError, step
from conftest import assert_close, make_prompts

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
NAMES = ["A", "B"]

_models = {}


def get_model(model_folders, name, dtype):
    key = (name, dtype)
    if key not in _models:
        _models[key] = Model.load(model_folders[name], dtype=dtype, device="cuda")
    return _models[key]


def logits_of(model, cache, entries):
    return step(model, cache, entries).float().cpu().numpy()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_each_request_alone_and_whole(model_folders, plain_logits, name, dtype):
    model = get_model(model_folders, name, dtype)
    cache = model.new_cache(max_tokens=64 * 8)
    for p in make_prompts(name, [1, 2, 5, 63, 64, 65, 200, 300]):
        slot = cache.open_sequence()
        got = logits_of(model, cache, [StepEntry(slot, p, list(range(len(p))))])
        assert_close(got, plain_logits(name, p), dtype, f"{name} {dtype} whole prompt of {len(p)}")
        cache.close_sequence(slot)
    assert cache.open_slots() == [] and cache.free_pages() == [8]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_last_32_tokens_one_by_one(model_folders, plain_logits, name, dtype):
    model = get_model(model_folders, name, dtype)
    cache = model.new_cache(max_tokens=64 * 4)
    for p in make_prompts(name, [33, 90, 160], seed=1):
        want = plain_logits(name, p)
        slot = cache.open_sequence()
        head = len(p) - 32
        got = [logits_of(model, cache, [StepEntry(slot, p[:head], list(range(head)))])]
        for t in range(head, len(p)):
            got.append(logits_of(model, cache, [StepEntry(slot, [p[t]], [0])]))
        assert_close(np.concatenate(got), want, dtype, f"{name} {dtype} {len(p)} tokens, last 32 decoded")
        cache.close_sequence(slot)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_one_after_another(model_folders, plain_logits, name, dtype):
    """Three batches through a cache that is too small to hold two of them at
    once: slots and pages of finished requests are used again, with the old
    keys still in them.  Within a batch each request is decoded up to its own
    length and leaves when it ends."""
    model = get_model(model_folders, name, dtype)
    cache = model.new_cache(max_tokens=64 * 7, max_slots=4)
    batches = [[(5, 9), (70, 3), (17, 20), (1, 12)], [(64, 1), (130, 6), (3, 33)], [(40, 8), (128, 2), (9, 9), (2, 2)]]
    for bi, batch in enumerate(batches):
        prompts = make_prompts(name, [a + b for a, b in batch], seed=10 + bi)
        want = [plain_logits(name, p) for p in prompts]
        slots = [cache.open_sequence() for _ in batch]
        got = [[] for _ in batch]
        # the prompts together, logits wanted at the last place only of the even
        # requests and everywhere for the odd ones
        entries = []
        for i, ((plen, _), p) in enumerate(zip(batch, prompts)):
            entries.append(StepEntry(slots[i], p[:plen], list(range(plen)) if i % 2 else [plen - 1]))
        flat = logits_of(model, cache, entries)
        o = 0
        for i, e in enumerate(entries):
            got[i].append((list(e.want), flat[o:o + len(e.want)]))
            o += len(e.want)
        # then one token each; a request that has had all its tokens leaves
        live = list(range(len(batch)))
        t = 0
        while live:
            live = [i for i in live if t < batch[i][1]]
            if not live:
                break
            entries = [StepEntry(slots[i], [prompts[i][batch[i][0] + t]], [0]) for i in live]
            flat = logits_of(model, cache, entries)
            for j, i in enumerate(live):
                got[i].append(([batch[i][0] + t], flat[j:j + 1]))
            for i in live:
                if t + 1 >= batch[i][1]:
                    cache.close_sequence(slots[i])      # ends earlier: its slot is free at once
            t += 1
        for i, pieces in enumerate(got):
            places = [pl for places, _ in pieces for pl in places]
            rows = np.concatenate([r for _, r in pieces])
            assert_close(rows, want[i][places], dtype, f"{name} {dtype} batch {bi} request {i}")
        assert cache.open_slots() == []
    assert cache.free_pages() == [7]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_long_decoding(model_folders, plain_logits, name, dtype):
    """A short prompt, then 330 tokens one by one across five page borders, next to
    a second request that leaves half-way."""
    model = get_model(model_folders, name, dtype)
    cache = model.new_cache(max_tokens=64 * 9)
    a, b = make_prompts(name, [7 + 330, 3 + 150], seed=3)
    wa, wb = plain_logits(name, a), plain_logits(name, b)
    sa, sb = cache.open_sequence(), cache.open_sequence()
    flat = logits_of(model, cache, [StepEntry(sa, a[:7], [6]), StepEntry(sb, b[:3], [2])])
    ga, gb = [flat[0:1]], [flat[1:2]]
    for t in range(330):
        entries = [StepEntry(sa, [a[7 + t]], [0])]
        if t < 150:
            entries.append(StepEntry(sb, [b[3 + t]], [0]))
        flat = logits_of(model, cache, entries)
        ga.append(flat[0:1])
        if t < 150:
            gb.append(flat[1:2])
        if t == 149:
            cache.close_sequence(sb)
    assert_close(np.concatenate(ga), wa[6:], dtype, f"{name} {dtype} long decode")
    assert_close(np.concatenate(gb), wb[2:], dtype, f"{name} {dtype} long decode, request that leaves")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_first_tokens_of_a_sequence(model_folders, plain_logits, name, dtype):
    """A one-token prompt is a prefill and a decode step at once; tokens 2..4 come
    one by one, in a batch with a request that starts with a longer prompt."""
    model = get_model(model_folders, name, dtype)
    cache = model.new_cache(max_tokens=64 * 4)
    p, other = make_prompts(name, [4, 70], seed=4)
    want = plain_logits(name, p)
    s, so = cache.open_sequence(), cache.open_sequence()
    got = [logits_of(model, cache, [StepEntry(s, p[:1], [0]), StepEntry(so, other[:66], [])])]
    for t in range(1, 4):
        got.append(logits_of(model, cache, [StepEntry(so, [other[66 + t - 1]], []), StepEntry(s, [p[t]], [0])]))
    assert_close(np.concatenate(got), want, dtype, f"{name} {dtype} first tokens")


@pytest.mark.parametrize("dtype", DTYPES)
def test_chunks_of_a_prompt(model_folders, plain_logits, dtype):
    """A prompt cut into runs of unequal size gives the logits of the whole."""
    name = "B"
    model = get_model(model_folders, name, dtype)
    cache = model.new_cache(max_tokens=64 * 4)
    (p,) = make_prompts(name, [150], seed=5)
    s = cache.open_sequence()
    got, o = [], 0
    for n in (1, 62, 1, 64, 22):
        got.append(logits_of(model, cache, [StepEntry(s, p[o:o + n], list(range(n)))]))
        o += n
    assert_close(np.concatenate(got), plain_logits(name, p), dtype, f"{dtype} chunked prompt")


def test_float32_cuttings_are_bitwise_equal(model_folders):
    """In the float32 path no reduction depends on the batch or on the cut, so
    whole, chunked and batched runs give identical bits."""
    name = "A"
    model = get_model(model_folders, name, "float32")
    cache = model.new_cache(max_tokens=64 * 8)
    p, q = make_prompts(name, [100, 37], seed=6)
    s = cache.open_sequence()
    whole = step(model, cache, [StepEntry(s, p, list(range(100)))]).clone()
    cache.close_sequence(s)
    s, s2 = cache.open_sequence(), cache.open_sequence()
    first = step(model, cache, [StepEntry(s2, q, [36]), StepEntry(s, p[:70], list(range(70)))])[1:].clone()
    rest = [step(model, cache, [StepEntry(s, [p[t]], [0]), StepEntry(s2, [q[0]], [])]).clone() for t in range(70, 100)]
    assert torch.equal(torch.cat([first] + rest), whole)


def test_step_refuses_bad_batches(model_folders):
    model = get_model(model_folders, "A", "float32")
    cache = model.new_cache(max_tokens=64 * 2)
    s = cache.open_sequence()
    with pytest.raises(StepError, match="vocabulary"):
        step(model, cache, [StepEntry(s, [256], [0])])
    with pytest.raises(StepError, match="twice"):
        step(model, cache, [StepEntry(s, [1], [0]), StepEntry(s, [2], [0])])
    with pytest.raises(StepError, match="not open"):
        step(model, cache, [StepEntry(3, [1], [0])])
    with pytest.raises(StepError, match="wanted place"):
        step(model, cache, [StepEntry(s, [1, 2], [2])])
    from go_tinygrad_b200.cache import CacheFull
    with pytest.raises(CacheFull):
        step(model, cache, [StepEntry(s, [1] * 129, [0])])
    assert cache.length(s) == 0 and cache.free_pages() == [2]      # nothing was taken
    assert step(model, cache, [StepEntry(s, [1, 2, 3], [])]).shape == (0, 256)
    assert cache.length(s) == 3


# ------------------------------------------------------------------ the per-op hook
OPS_OF_A_LAYER = ["hidden_in", "normed", "q", "k", "v", "q_attn", "attn", "o", "mlp_input",
                  "gate_pre", "up", "gate_act", "down", "hidden_post_ffn"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_the_op_hook_names_every_value_of_a_layer(model_folders, plain_models, name, dtype):
    """With `model.op_hook` set, every layer hands its named intermediate values to
    the hook, under the reference's names; the plain implementation emits the same
    names, and the two are compared op by op -- the tool that says WHERE a model
    that drifts starts to drift.  Without a hook nothing is called, and decode
    steps of a generation are recorded as graphs again."""
    import plain_llama
    from go_tinygrad_b200.engine.generate import generate
    model = Model.load(model_folders[name], dtype=dtype, device="cuda")
    cfg, w = plain_models[name]
    (p,) = make_prompts(name, [37], seed=21)
    want = {}
    plain_llama.forward(cfg, w, p, trace=lambda layer, op, value: want.__setitem__((layer, op), np.array(value)))
    got, steps = {}, set()

    def hook(step_index, layer, op, tensor):
        steps.add(step_index)
        got[(layer, op)] = tensor.float().cpu().numpy()
    model.op_hook = hook
    cache = model.new_cache(max_tokens=64 * 2)
    slot = cache.open_sequence()
    first = model.steps_run
    step(model, cache, [StepEntry(slot, p, [len(p) - 1])])
    assert steps == {first}
    n_layers = cfg["num_hidden_layers"]
    expected = set(OPS_OF_A_LAYER)
    if dtype == "bfloat16" and cfg["intermediate_size"] % 8 == 0:
        expected -= {"gate_pre", "up"}               # the activation is applied in the product's epilogue
    assert {op for (layer, op) in got} == expected and {layer for (layer, op) in got} == set(range(n_layers))
    for (layer, op), value in got.items():
        ref = want[(layer, op)]
        assert value.shape == ref.shape, (layer, op)
        limit = (2e-5 if dtype == "float32" else 3e-2) * max(1.0, float(np.abs(ref).max()))
        assert np.abs(value - ref).max() <= limit, f"layer {layer} {op}: {np.abs(value - ref).max():.3e} > {limit:.3e}"
    # a decode step under the hook runs in the open and reports its one token
    got.clear()
    assert not model.capturable
    out = generate(model, [p[:9]], max_new_tokens=3, stop=[])
    assert len(out[0].tokens) == 3 and got[(0, "normed")].shape == (1, cfg["hidden_size"])
    model.op_hook = None
    got.clear()
    assert model.capturable
    again = generate(model, [p[:9]], max_new_tokens=3, stop=[])
    assert [r.tokens for r in again] == [r.tokens for r in out] and not got
    cache.close_sequence(slot)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_step_of_a_size_that_has_run_asks_the_allocator_for_its_result_only(model_folders, plain_logits, dtype):
    """The intermediates of a step come from the model's workspace.  Once a step of a
    size has run, the same step again makes the allocator hand out its result and
    nothing else, whatever the number of layers; its logits are the same bits, and
    logits kept from an earlier step are not touched by a later one."""
    model = Model.load(model_folders["A"], dtype=dtype, device="cuda")
    cache = model.new_cache(max_tokens=64 * 4)
    (p,) = make_prompts("A", [45], seed=31)
    count = lambda: torch.cuda.memory_stats()["allocation.all.allocated"]

    def prompt_then_two_tokens():
        slot = cache.open_sequence()
        out, asked = [], []
        for tokens in (p[:43], p[43:44], p[44:45]):
            before = count()
            out.append(step(model, cache, [StepEntry(slot, tokens, [len(tokens) - 1])]))
            asked.append(count() - before)
        cache.close_sequence(slot)
        return out, asked
    first, _ = prompt_then_two_tokens()
    kept = [t.clone() for t in first]
    prompt_then_two_tokens()
    again, asked = prompt_then_two_tokens()
    assert asked == [1, 1, 1], f"allocations per step: {asked}"
    for a, b, c in zip(first, kept, again):
        assert torch.equal(a, b) and torch.equal(a, c)
    assert len(model.rt.workspace.buffers()) == 3
    want = plain_logits("A", p)
    got = torch.cat(again).float().cpu().numpy()
    assert_close(got, want[[42, 43, 44]], dtype, "steps from the workspace")
