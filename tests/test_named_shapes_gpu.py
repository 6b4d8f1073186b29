"""The layer shapes of the models the reference's engine names (SmolLM2-1.7B,
Llama-3.2-1B, Llama-3.1-8B): one layer of each with its true widths, head counts,
head size, grouping and rotary scaling, and a small vocabulary, against the plain
implementation in float32 and in bfloat16.  The tiny configurations elsewhere pick
sizes that are awkward on purpose; these are the sizes the kernels are tuned for
(inner sizes of 8192 and 14336 split over clusters, heads of 128 channels, four
query heads per key/value head), which a tiny model never reaches."""
import numpy as np
import pytest

import go_tinygrad_b200 as lib
from go_tinygrad_b200.engine import Model, StepEntry, step
from conftest import assert_close

pytestmark = pytest.mark.gpu

LLAMA3 = {"rope_type": "llama3", "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 8192}
BASE = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 1,
        "rms_norm_eps": 1e-5, "max_position_embeddings": 8192}
SHAPES = {
    "smollm2-1.7b": dict(BASE, hidden_size=2048, num_attention_heads=32, num_key_value_heads=32, head_dim=64,
                         intermediate_size=8192, vocab_size=1000, rope_theta=130000.0, rope_scaling=None,
                         tie_word_embeddings=True),
    "llama-3.2-1b": dict(BASE, hidden_size=2048, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
                         intermediate_size=8192, vocab_size=1000, rope_theta=500000.0,
                         rope_scaling=dict(LLAMA3, factor=32.0), tie_word_embeddings=True),
    "llama-3.1-8b": dict(BASE, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                         intermediate_size=14336, vocab_size=1000, rope_theta=500000.0,
                         rope_scaling=dict(LLAMA3, factor=8.0), tie_word_embeddings=False),
}
PROMPTS, DECODED = (70, 17, 130), 6


@pytest.fixture(scope="module")
def shape_cases(tmp_path_factory):
    """name -> (folder, requests, the plain implementation's logits for each request)."""
    import plain_llama
    out = {}
    rng = np.random.default_rng(11)
    for name, cfg in SHAPES.items():
        folder = str(tmp_path_factory.mktemp(name.replace(".", "_")))
        lib.write_random_model(folder, cfg, seed=3, dtype="bfloat16", std=0.02, norm_std=0.05)
        pcfg, w = plain_llama.read_model(folder)
        requests = [rng.integers(0, cfg["vocab_size"], n + DECODED).tolist() for n in PROMPTS]
        out[name] = (folder, requests, [plain_llama.forward(pcfg, w, r) for r in requests])
        del w
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(SHAPES))
def test_prompts_in_one_step_then_token_by_token(shape_cases, name, dtype):
    folder, requests, want = shape_cases[name]
    model = Model.load(folder, dtype=dtype, device="cuda")
    cache = model.new_cache(max_tokens=64 * 8)
    slots = [cache.open_sequence() for _ in requests]
    got = [[] for _ in requests]
    logits = step(model, cache, [StepEntry(s, r[:n], list(range(n))) for s, r, n in zip(slots, requests, PROMPTS)])
    at = 0
    for i, n in enumerate(PROMPTS):
        got[i].append(logits[at:at + n].float().cpu().numpy())
        at += n
    live = list(range(len(requests)))
    for t in range(DECODED):
        if t == DECODED - 2:                       # the shortest request ends two tokens early
            cache.close_sequence(slots[1])
            live.remove(1)
        logits = step(model, cache, [StepEntry(slots[i], [requests[i][PROMPTS[i] + t]], [0]) for i in live])
        for row, i in enumerate(live):
            got[i].append(logits[row:row + 1].float().cpu().numpy())
    for i in range(len(requests)):
        have = np.concatenate(got[i])
        assert_close(have, want[i][:len(have)], dtype, f"{name} {dtype} request {i}")
    from go_tinygrad_b200.kernels import ops
    assert ops.bounded_wait_failures() == 0


@pytest.mark.parametrize("name", ["smollm2-1.7b", "llama-3.1-8b"])
def test_decode_steps_of_more_sequences_than_the_streaming_products_take(shape_cases, name):
    """70 sequences: their decode steps have more rows than the weight-streaming
    products take, so the prompt-sized products (and, at 64 channels, the projection
    that rotates and stores in its epilogue) run in a decode step."""
    import plain_llama
    folder = shape_cases[name][0]
    pcfg, w = plain_llama.read_model(folder)
    rng = np.random.default_rng(5)
    n_seqs, decoded = 70, 2
    lengths = rng.integers(3, 9, n_seqs).tolist()
    requests = [rng.integers(0, pcfg["vocab_size"], n + decoded).tolist() for n in lengths]
    model = Model.load(folder, dtype="bfloat16", device="cuda")
    cache = model.new_cache(max_tokens=64 * n_seqs, max_slots=n_seqs)
    slots = [cache.open_sequence() for _ in requests]
    step(model, cache, [StepEntry(s, r[:n], []) for s, r, n in zip(slots, requests, lengths)])
    got = []
    for t in range(decoded):
        logits = step(model, cache, [StepEntry(s, [r[n + t]], [0]) for s, r, n in zip(slots, requests, lengths)])
        got.append(logits.float().cpu().numpy())
    for i in (0, 1, 33, 68, 69):
        want = plain_llama.forward(pcfg, w, requests[i])
        have = np.stack([got[t][i] for t in range(decoded)])
        assert_close(have, want[lengths[i]:lengths[i] + decoded], "bfloat16", f"{name} sequence {i} of {n_seqs}")
