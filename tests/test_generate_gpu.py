"""Generation through the Python entry point and the command line: greedy and
temperature sampling against the plain implementation, stop tokens, sequences
that end earlier, and batch after batch through one small cache."""
import os
import subprocess
import sys

import numpy as np
import pytest

import go_tinygrad_b200 as lib
import plain_llama
from conftest import ROOT, TINY, make_prompts

pytestmark = pytest.mark.gpu

_models = {}


def get_model(model_folders, name, dtype):
    if (name, dtype) not in _models:
        _models[(name, dtype)] = lib.Model.load(model_folders[name], dtype=dtype, device="cuda")
    return _models[(name, dtype)]


def check_tokens(plain_models, name, prompt, tokens, dtype, temperature=0.0, seed=0, request=0):
    """Every generated token must be one the plain implementation could have
    chosen from the same prefix: the maximum (or a logit within rounding of it),
    or the token whose cumulative-probability interval holds the draw."""
    cfg, w = plain_models[name]
    seq = list(prompt)
    for step, tok in enumerate(tokens):
        logits = plain_llama.forward(cfg, w, seq)[-1].astype(np.float64)
        slack = (1e-4 if dtype == "float32" else 5e-2) * max(1.0, np.abs(logits).max())
        if temperature == 0.0:
            assert logits[tok] >= logits.max() - slack, (step, tok, int(logits.argmax()))
            if dtype == "float32":
                assert tok == plain_llama.argmax_first(logits.astype(np.float32))
        else:
            u = plain_llama.uniform(seed, request, step)
            cdf = np.cumsum(plain_llama.temperature_probs(logits, temperature))
            eps = 1e-5 if dtype == "float32" else 3e-2
            below = cdf[tok - 1] if tok > 0 else 0.0
            assert below - eps <= u <= cdf[tok] + eps, (step, tok, u, below, cdf[tok])
        seq.append(tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation(model_folders, plain_models, name, dtype):
    model = get_model(model_folders, name, dtype)
    prompts = make_prompts(name, [5, 17, 32, 1], seed=31)
    results = lib.generate(model, prompts, 16, stop=[])
    assert [r.finish_reason for r in results] == ["length"] * 4
    for i, (p, r) in enumerate(zip(prompts, results)):
        assert len(r.tokens) == 16
        check_tokens(plain_models, name, p, r.tokens, dtype)
    if dtype == "float32":
        cfg, w = plain_models[name]
        assert results[1].tokens == plain_llama.generate(cfg, w, prompts[1], 16)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_temperature_sampling(model_folders, plain_models, dtype):
    name = "B"
    model = get_model(model_folders, name, dtype)
    prompts = make_prompts(name, [1, 9, 40, 64], seed=32)
    results = model.generate(prompts, 24, temperature=0.8, seed=7, stop=[])
    for i, (p, r) in enumerate(zip(prompts, results)):
        check_tokens(plain_models, name, p, r.tokens, dtype, temperature=0.8, seed=7, request=i)
    # another seed draws other tokens; the same seed the same
    again = model.generate(prompts, 24, temperature=0.8, seed=7, stop=[])
    other = model.generate(prompts, 24, temperature=0.8, seed=8, stop=[])
    assert [r.tokens for r in again] == [r.tokens for r in results] != [r.tokens for r in other]


def test_stop_tokens_and_earlier_ends_leave_the_others_alone(model_folders, plain_models):
    name = "A"
    model = get_model(model_folders, name, "float32")
    prompts = make_prompts(name, [6, 70, 3, 20, 9], seed=33)
    free = lib.generate(model, prompts, 12, stop=[])
    # stop on a token that request 1 produces early; per-request limits differ
    stop = free[1].tokens[2]
    limits = [12, 12, 4, 0, 7]
    results = lib.generate(model, prompts, limits, stop=[stop])
    for f, r, limit in zip(free, results, limits):
        want = f.tokens[:limit]
        if stop in want:
            want = want[:want.index(stop) + 1]
            assert r.finish_reason == "stop"
        else:
            assert r.finish_reason == "length"
        assert r.tokens == want          # float32: what else runs in the batch changes nothing
    assert results[3].tokens == []
    # the model's own end tokens are the default stop set
    cfg, w = plain_models[name]
    eos = TINY[name]["eos_token_id"]
    default = lib.generate(model, prompts, 12)
    for f, r in zip(free, default):
        want = f.tokens[:f.tokens.index(eos) + 1] if eos in f.tokens else f.tokens
        assert r.tokens == want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_generation_with_members_that_leave_and_recordings_made_again(model_folders, plain_models, dtype):
    """Sequences grow to many times their prompts (the recorded decode step is
    planned for a length and made again when outgrown) and end at different
    times (a recording is kept per batch size and given other slots): the
    replayed graphs must produce what launching kernel by kernel produces."""
    name = "B"
    model = get_model(model_folders, name, dtype)
    prompts = make_prompts(name, [3, 40, 17, 1, 9], seed=35)
    limits = [150, 60, 150, 20, 100]
    graphs = lib.generate(model, prompts, limits, stop=[])
    eager = lib.generate(model, prompts, limits, stop=[], use_graph=False)
    assert [len(r.tokens) for r in graphs] == limits == [len(r.tokens) for r in eager]
    if dtype == "float32":              # no sum depends on the recording's plan: the same tokens
        assert [r.tokens for r in graphs] == [r.tokens for r in eager]
    for i in (0, 1, 4):
        check_tokens(plain_models, name, prompts[i], graphs[i].tokens[:48], dtype)


def test_batch_after_batch_through_a_small_cache(model_folders):
    name = "B"
    model = get_model(model_folders, name, "float32")
    prompts = make_prompts(name, [30, 100, 5, 64, 2, 90, 17], seed=34)
    alone = [lib.generate(model, [p], 10, stop=[], temperature=0.7, seed=3)[0] for p in prompts]
    cache = model.new_cache(max_tokens=64 * 4, max_slots=3)
    together = lib.generate(model, prompts, 10, stop=[], temperature=0.7, seed=3, cache=cache)
    # a request's draws are keyed by its index among the requests of the call
    for i, (p, r) in enumerate(zip(prompts, together)):
        solo = lib.generate(model, [[0]] * i + [p], [0] * i + [10], stop=[], temperature=0.7, seed=3)[i]
        assert r.tokens == solo.tokens
    assert alone[0].tokens == together[0].tokens
    assert cache.open_slots() == [] and cache.free_pages() == [4]


def test_a_cache_kept_over_calls_keeps_its_recorded_decode_steps(model_folders, monkeypatch):
    """The decode batches a call of `generate` makes stay with a cache the caller owns: a
    second call with that cache builds none, whatever its prompts, and gives what a call
    on a cache of its own gives; another temperature is another recording."""
    from go_tinygrad_b200.engine import generate as generate_module
    name = "A"
    model = get_model(model_folders, name, "bfloat16")
    made = []
    real = generate_module.DecodeBatch

    def counting(*args, **kwargs):
        made.append(1)
        return real(*args, **kwargs)
    monkeypatch.setattr(generate_module, "DecodeBatch", counting)
    cache = model.new_cache(max_tokens=64 * 8, max_slots=3)
    first_prompts = make_prompts(name, [40, 9, 70], seed=51)
    second_prompts = make_prompts(name, [5, 120, 33], seed=52)
    limits = [12, 5, 9]                                       # sizes 3, 2 and 1 each get a recording
    lib.generate(model, first_prompts, limits, stop=[], cache=cache)
    assert len(made) == 3 and len(cache.attachments["decode_batches"]) == 3
    second = lib.generate(model, second_prompts, limits, stop=[], cache=cache)
    assert len(made) == 3, "the second call made decode batches of its own"
    fresh = lib.generate(model, second_prompts, limits, stop=[])
    assert [r.tokens for r in second] == [r.tokens for r in fresh]
    lib.generate(model, second_prompts, limits, stop=[], cache=cache, temperature=0.5, seed=1)
    assert len(made) == 6 + 3                                 # the call on its own cache, and the other temperature
    assert cache.open_slots() == []


def test_command_line(model_folders, plain_models):
    name = "A"
    cfg, w = plain_models[name]
    prompt = make_prompts(name, [9], seed=35)[0]
    want = plain_llama.generate(cfg, w, prompt, 8)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "llmgen"), "-model", model_folders[name],
                          "-ids", ",".join(map(str, prompt)), "-ids", "7 8 9", "-tokens", "8", "-gpu",
                          "-dtype", "float32", "-stop", "999"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    assert f"[0] ids: {' '.join(map(str, want))}  (length)" in out.stdout
    assert "Prompt tokens:    12" in out.stdout and "Generated tokens: 16" in out.stdout
    bad = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "llmgen"), "-model", model_folders[name],
                          "-tokens", "-1"], capture_output=True, text=True, timeout=300)
    assert bad.returncode == 1 and "non-negative" in bad.stderr
