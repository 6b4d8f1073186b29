"""The two tiny configurations and workloads exactly as the benchmark description
names them: tiny-llama-A (2 layers, width 64, 4 heads on 2, heads of 16, 128/256,
plain rotation, tied head; weights N(0, 0.02), norms 1 + N(0, 0.01), seed 0; prompts
of 5, 17 and 32 tokens, 16 greedy steps) and tiny-llama-B (3 layers, width 96, 3
heads on 1, heads of 32, 256/384, llama3-scaled rotation, separate head; N(0, 0.03),
1 + N(0, 0.02), seed 1; prompts of 1, 9, 40 and 64 tokens, 24 steps at temperature
0.8 with seed 7), in float32 against the plain implementation and in bfloat16
against the float32 logits' tolerance."""
import numpy as np
import pytest

import go_tinygrad_b200 as lib
import plain_llama
from go_tinygrad_b200.engine import StepEntry, step
from conftest import NAMED_TINY, assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", list(NAMED_TINY))
def test_the_named_tiny_workloads(tmp_path, name):
    raw, seed, std, norm_std, lengths, steps, temperature, sample_seed = NAMED_TINY[name]
    folder = str(tmp_path / "m")
    lib.write_random_model(folder, raw, seed=seed, dtype="float32", std=std, norm_std=norm_std)
    cfg, w = plain_llama.read_model(folder)
    rng = np.random.default_rng(seed)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in lengths]
    model = lib.Model.load(folder, dtype="float32", device="cuda")
    got = lib.generate(model, prompts, max_new_tokens=steps, temperature=temperature, seed=sample_seed, stop=[])
    for i, (p, r) in enumerate(zip(prompts, got)):
        assert len(r.tokens) == steps
        # judged token by token on the sequence the engine itself produced: the plain
        # logits there must choose (or, with a temperature, draw) the same token
        logits = plain_llama.forward(cfg, w, p + r.tokens)
        for t, tok in enumerate(r.tokens):
            row = logits[len(p) - 1 + t]
            if temperature > 0:
                u = plain_llama.uniform(sample_seed, i, t)
                cdf = np.cumsum(plain_llama.temperature_probs(row, temperature))
                below = cdf[tok - 1] if tok > 0 else 0.0
                assert below - 1e-5 <= u <= cdf[tok] + 1e-5, f"{name}: request {i}, token {t}"
            else:
                top2 = np.partition(row, -2)[-2:]
                if top2[1] - top2[0] > 1e-5:
                    assert tok == int(np.argmax(row)), f"{name}: request {i}, token {t}"
    # the same requests through the step function, both precisions: prompts together, then one token each
    requests = [p + r.tokens for p, r in zip(prompts, got)]
    want = [plain_llama.forward(cfg, w, r) for r in requests]
    for dtype in ("float32", "bfloat16"):
        m = model if dtype == "float32" else lib.Model.load(folder, dtype=dtype, device="cuda")
        cache = m.new_cache(max_tokens=64 * 2 * len(requests), max_slots=len(requests))
        slots = [cache.open_sequence() for _ in requests]
        out = step(m, cache, [StepEntry(s, r[:n], list(range(n))) for s, r, n in zip(slots, requests, lengths)])
        out = out.float().cpu().numpy()
        o = 0
        for i, n in enumerate(lengths):
            assert_close(out[o:o + n], want[i][:n], dtype, f"{name} {dtype}: prompt {i}")
            o += n
        for t in range(steps):
            out = step(m, cache, [StepEntry(s, [r[n + t]], [0]) for s, r, n in zip(slots, requests, lengths)])
            out = out.float().cpu().numpy()
            for i, n in enumerate(lengths):
                assert_close(out[i], want[i][n + t], dtype, f"{name} {dtype}: step {t} of request {i}")
