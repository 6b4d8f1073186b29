"""The engine at the layer sizes of the models it is measured on (SmolLM2-1.7B,
Llama-3.2-1B, Llama-3.1-8B), with one or two layers and a small vocabulary so
that the plain implementation stays cheap.  These shapes reach the kernels the
tiny configurations do not: the tcgen05 product, cluster-split rows of 8192 and
14336, heads of 128, groups of four query heads per key/value head."""
import math

import numpy as np
import pytest

import go_tinygrad_b200 as lib
import plain_llama
from go_tinygrad_b200.engine import StepEntry, step

pytestmark = pytest.mark.gpu

LLAMA3 = lambda factor: {"rope_type": "llama3", "factor": factor, "low_freq_factor": 1.0,
                         "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}
BASE = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "rms_norm_eps": 1e-5,
        "max_position_embeddings": 8192}
SHAPES = {
    "smollm2": dict(BASE, num_hidden_layers=2, hidden_size=2048, num_attention_heads=32, num_key_value_heads=32,
                    head_dim=64, intermediate_size=8192, vocab_size=4096, rope_theta=130000.0, rope_scaling=None,
                    tie_word_embeddings=True),
    "llama32": dict(BASE, num_hidden_layers=1, hidden_size=2048, num_attention_heads=32, num_key_value_heads=8,
                    head_dim=64, intermediate_size=8192, vocab_size=4099, rope_theta=500000.0,
                    rope_scaling=LLAMA3(32.0), tie_word_embeddings=True),
    "llama31": dict(BASE, num_hidden_layers=1, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                    head_dim=128, intermediate_size=14336, vocab_size=4000, rope_theta=500000.0,
                    rope_scaling=LLAMA3(8.0), tie_word_embeddings=False),
}


@pytest.fixture(scope="module", params=list(SHAPES))
def shaped(request, tmp_path_factory):
    name = request.param
    folder = str(tmp_path_factory.mktemp(f"shape_{name}"))
    lib.write_random_model(folder, SHAPES[name], seed=11, dtype="bfloat16", std=0.02, norm_std=0.05)
    cfg, w = plain_llama.read_model(folder)
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (150, 70)]
    want = [plain_llama.forward(cfg, w, p) for p in prompts]
    return name, folder, prompts, want


def check(got, want, dtype, widest, what):
    """Dot products of `widest` terms: float32 rounding grows with its square root."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert np.isfinite(got).all(), what
    scale = max(1.0, np.abs(want).max())
    err = np.abs(got - want)
    if dtype == "float32":
        lim_max, lim_mean = 5e-5 * scale * math.sqrt(widest / 256), 5e-6 * scale * math.sqrt(widest / 256)
    else:
        lim_max, lim_mean = 5e-2 * scale, 6e-3 * scale
    assert err.max() <= lim_max and err.mean() <= lim_mean, \
        f"{what}: max {err.max():.3e} (limit {lim_max:.3e}), mean {err.mean():.3e} (limit {lim_mean:.3e})"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_layer_shapes(shaped, dtype):
    name, folder, prompts, want = shaped
    widest = SHAPES[name]["intermediate_size"]
    model = lib.Model.load(folder, dtype=dtype, device="cuda")
    cache = model.new_cache(max_tokens=64 * 6)
    slots = [cache.open_sequence() for _ in prompts]
    # the prompts without their last four tokens, together; then one token each
    heads = [len(p) - 4 for p in prompts]
    got = step(model, cache, [StepEntry(s, p[:h], [0, h // 2, h - 1]) for s, p, h in zip(slots, prompts, heads)])
    got = got.float().cpu().numpy()
    for i, (w, h) in enumerate(zip(want, heads)):
        check(got[3 * i: 3 * i + 3], w[[0, h // 2, h - 1]], dtype, widest, f"{name} {dtype} prompt {i}")
    for t in range(4):
        got = step(model, cache, [StepEntry(s, [p[h + t]], [0]) for s, p, h in zip(slots, prompts, heads)])
        got = got.float().cpu().numpy()
        for i, (w, h) in enumerate(zip(want, heads)):
            check(got[i], w[h + t], dtype, widest, f"{name} {dtype} decoded token {t} of prompt {i}")
    from go_tinygrad_b200.kernels import ops
    assert ops.bounded_wait_failures() == 0


def test_decode_steps_of_more_sequences_than_the_streaming_products_take(shaped):
    """70 sequences: their decode steps have more rows than the weight-streaming
    products take, so the prompt-sized products (and, at 64 channels, the projection
    that rotates and stores in its epilogue) run in a decode step."""
    name, folder, _, _ = shaped
    cfg, w = plain_llama.read_model(folder)
    rng = np.random.default_rng(5)
    n_seqs, decoded = 70, 2
    lengths = rng.integers(3, 9, n_seqs).tolist()
    requests = [rng.integers(0, cfg["vocab_size"], n + decoded).tolist() for n in lengths]
    model = lib.Model.load(folder, dtype="bfloat16", device="cuda")
    cache = model.new_cache(max_tokens=64 * n_seqs, max_slots=n_seqs)
    slots = [cache.open_sequence() for _ in requests]
    step(model, cache, [StepEntry(s, r[:n], []) for s, r, n in zip(slots, requests, lengths)])
    got = []
    for t in range(decoded):
        logits = step(model, cache, [StepEntry(s, [r[n + t]], [0]) for s, r, n in zip(slots, requests, lengths)])
        got.append(logits.float().cpu().numpy())
    for i in (0, 1, 33, 68, 69):
        want = plain_llama.forward(cfg, w, requests[i])
        have = np.stack([got[t][i] for t in range(decoded)])
        check(have, want[lengths[i]:lengths[i] + decoded], "bfloat16", cfg["intermediate_size"], f"{name} sequence {i} of {n_seqs}")


def test_keys_in_the_cache_depend_on_the_cutting_within_rounding_only(shaped):
    """In bfloat16 a token's key is rounded where it is made, and prompts, short chunks
    and single tokens make it in different kernels (rotation on the float accumulators
    of the prompt projection; on the rounded projection in steps of up to 64 rows and
    inside the decode attention).  The same 130 tokens fed whole, as 40 + 90 and as 129
    + 1 must leave the same keys and values up to that rounding.  The first layer's inputs
    are identical; a rotated channel a cos - b sin inherits the rounding of both a and b,
    so the bound is three units of the last place of the head's largest channel (values,
    which are not rotated: of the value itself)."""
    import torch
    name, folder, prompts, _ = shaped
    tokens = prompts[0][:130]
    model = lib.Model.load(folder, dtype="bfloat16", device="cuda")

    def run(cuts):
        cache = model.new_cache(max_tokens=64 * 3, max_slots=1)
        slot = cache.open_sequence()
        done = 0
        for n in cuts:
            step(model, cache, [StepEntry(slot, tokens[done:done + n], [])])
            done += n
        t = torch.arange(done)
        pages = cache.groups[0].table_host[slot][t // 64].long().cuda()
        out = []
        for entry in (0, len(model.plan.schedule) - 1):
            kv = cache.handles[entry].kv
            out.append((kv.k[pages, :, (t % 64).cuda(), :].float(), kv.v[pages, :, (t % 64).cuda(), :].float()))
        return out
    whole, chunks, last_alone = run([130]), run([40, 90]), run([129, 1])
    for other, what in ((chunks, "40 + 90"), (last_alone, "129 + 1")):
        (k0, v0), (k1, v1) = whole[0], other[0]                 # the first layer: same inputs, other kernels
        ulp = 2.0 ** -8
        for a, b, which in ((k0, k1, "keys"), (v0, v1, "values")):
            size = a.abs().amax(dim=-1, keepdim=True) if which == "keys" else torch.maximum(a.abs(), b.abs())
            worst = float(((a - b).abs() / (size + 1e-3)).max())
            assert worst <= 3 * ulp, f"{name}: first layer's {which}, whole against {what}: {worst / ulp:.2f} units"
        (k0, v0), (k1, v1) = whole[1], other[1]                 # the last layer: its inputs carry the rounding on
        for a, b in ((k0, k1), (v0, v1)):
            assert float((a - b).abs().max()) <= 5e-2 * max(1.0, float(a.abs().max()))
