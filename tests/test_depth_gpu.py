"""Parity at depth and at the real vocabularies: the whole SmolLM2-1.7B shape (24
layers, 49,152 entries), the whole Llama-3.2-1B shape (16 layers, 128,256 entries,
llama3 frequency scaling by 32) and four layers of the Llama-3.1-8B shape (heads of
128, a separate head of 128,256 entries), with random weights, in float32 and in
bfloat16, against the plain implementation: a prompt whole, its last eight tokens
one by one, an unequal batch of three whose shorter requests end earlier, and greedy
generation through the entry point.

The tolerance in float32 does not grow with depth: the engine and the plain
implementation differ in the order of their sums only, and the residual stream
carries those differences forward without amplifying them (every layer's input is
normalised).  Every comparison keeps the bound the shallow tests use (5e-5 of the
largest logit times the square root of (widest dot product / 256)), and over all
cuttings together the largest float32 error must stay below 5e-5 of the largest
logit outright (measured: 1.4e-5 at 24 layers, 1.7e-5 at four layers of width
4,096).  One module-scoped model folder per shape is written to a temporary place
and read by both sides."""
import math
import os

import numpy as np
import pytest
import torch

import go_tinygrad_b200 as lib
import plain_llama
from go_tinygrad_b200.config.registry import find_architecture
from go_tinygrad_b200.engine import StepEntry, step
from go_tinygrad_b200.parts.plan import plan_weight_specs
from go_tinygrad_b200.weights import random_tensors, write_safetensors
from test_real_shapes_gpu import BASE, LLAMA3, check as check_logits

pytestmark = pytest.mark.gpu

DEEP = {
    "smollm2-1.7b": dict(BASE, num_hidden_layers=24, hidden_size=2048, num_attention_heads=32, num_key_value_heads=32,
                         head_dim=64, intermediate_size=8192, vocab_size=49152, rope_theta=130000.0, rope_scaling=None,
                         tie_word_embeddings=True),
    "llama-3.2-1b": dict(BASE, num_hidden_layers=16, hidden_size=2048, num_attention_heads=32, num_key_value_heads=8,
                         head_dim=64, intermediate_size=8192, vocab_size=128256, rope_theta=500000.0,
                         rope_scaling=LLAMA3(32.0), tie_word_embeddings=True, max_position_embeddings=131072),
    "llama-3.1-8b/4": dict(BASE, num_hidden_layers=4, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                           head_dim=128, intermediate_size=14336, vocab_size=128256, rope_theta=500000.0,
                           rope_scaling=LLAMA3(8.0), tie_word_embeddings=False, max_position_embeddings=131072),
}
LENGTHS = (40, 23, 9)          # the requests of the unequal batch; the first is also run alone
NEW_TOKENS = 4


def write_folder(folder, raw, seed):
    """config.json and model.safetensors with weights drawn on the GPU (a billion
    values and more: the host's generator would take most of the test's time)."""
    import json
    arch = find_architecture(raw)
    specs = plan_weight_specs(arch.plan(arch.read_config(raw)))
    tensors = random_tensors(specs, seed, 0.02, 0.05, torch.bfloat16, device="cuda")
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)


@pytest.fixture(scope="module", params=list(DEEP))
def deep(request, tmp_path_factory):
    name = request.param
    folder = str(tmp_path_factory.mktemp("deep"))
    write_folder(folder, DEEP[name], seed=31)
    cfg, w = plain_llama.read_model(folder)
    rng = np.random.default_rng(9)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in LENGTHS]
    # greedy continuation by the float32 engine; the plain implementation then runs
    # prompt + continuation once per request and judges every token of it
    model = lib.Model.load(folder, dtype="float32", device="cuda")
    generated = [r.tokens for r in lib.generate(model, prompts, max_new_tokens=NEW_TOKENS, stop=[])]
    del model
    torch.cuda.empty_cache()
    requests = [p + g for p, g in zip(prompts, generated)]
    want = [plain_llama.forward(cfg, w, r) for r in requests]
    del w
    yield name, folder, cfg, prompts, generated, requests, want
    for f in os.listdir(folder):
        os.remove(os.path.join(folder, f))


def test_greedy_generation_at_depth_matches_the_plain_implementation(deep):
    name, folder, cfg, prompts, generated, requests, want = deep
    for i, (p, g) in enumerate(zip(prompts, generated)):
        assert len(g) == NEW_TOKENS
        for t, tok in enumerate(g):
            row = want[i][len(p) - 1 + t]
            best = int(np.argmax(row))
            top2 = np.partition(row, -2)[-2:]
            if top2[1] - top2[0] > 1e-3 * max(1.0, float(np.abs(row).max())):    # a clear winner must be the token taken
                assert tok == best, f"{name}: request {i}, new token {t}: engine {tok}, plain {best}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_cutting_at_depth_and_real_vocabulary(deep, dtype):
    name, folder, cfg, prompts, generated, requests, want = deep
    widest = cfg["intermediate_size"]
    model = lib.Model.load(folder, dtype=dtype, device="cuda")
    cache = model.new_cache(max_tokens=64 * 4, max_slots=3)
    logits = lambda entries: step(model, cache, entries).float().cpu().numpy()
    worst = {"max": 0.0, "mean": 0.0}

    def check(got, want, dtype, widest, what):
        check_logits(got, want, dtype, widest, what)
        scale = max(1.0, float(np.abs(want).max()))
        err = np.abs(np.asarray(got, np.float64) - np.asarray(want, np.float64))
        worst["max"], worst["mean"] = max(worst["max"], err.max() / scale), max(worst["mean"], err.mean() / scale)

    # the first request whole, logits everywhere
    r = requests[0]
    slot = cache.open_sequence()
    got = logits([StepEntry(slot, r, list(range(len(r))))])
    check(got, want[0], dtype, widest, f"{name} {dtype}: whole")
    cache.close_sequence(slot)

    # its last eight tokens one by one
    slot = cache.open_sequence()
    head = len(r) - 8
    got = [logits([StepEntry(slot, r[:head], [head - 1])])]
    for t in range(head, len(r)):
        got.append(logits([StepEntry(slot, [r[t]], [0])]))
    check(np.concatenate(got), want[0][head - 1:], dtype, widest, f"{name} {dtype}: last eight one by one")
    cache.close_sequence(slot)

    # the unequal batch: prompts together, then one token each; the shorter end earlier
    slots = [cache.open_sequence() for _ in requests]
    got = logits([StepEntry(s, r[:n], [n - 1]) for s, r, n in zip(slots, requests, LENGTHS)])
    for i, n in enumerate(LENGTHS):
        check(got[i], want[i][n - 1], dtype, widest, f"{name} {dtype}: batch, prompt {i}")
    live = list(range(len(requests)))
    for t in range(NEW_TOKENS):
        if t == 2:                                        # the shortest request leaves after two tokens
            cache.close_sequence(slots[2])
            live = [0, 1]
        got = logits([StepEntry(slots[i], [requests[i][LENGTHS[i] + t]], [0]) for i in live])
        for row, i in enumerate(live):
            check(got[row], want[i][LENGTHS[i] + t], dtype, widest, f"{name} {dtype}: batch, token {t} of request {i}")
    for i in live:
        cache.close_sequence(slots[i])
    assert cache.open_slots() == []
    print(f"{name} {dtype}: largest error over all cuttings, relative to the largest logit: "
          f"max {worst['max']:.2e}, mean {worst['mean']:.2e}")
    if dtype == "float32":
        assert worst["max"] <= 5e-5 and worst["mean"] <= 1e-5, worst
    from go_tinygrad_b200.kernels import ops
    assert ops.bounded_wait_failures() == 0
