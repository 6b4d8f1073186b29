"""Shared test set-up: the `gpu` marker, the two tiny configurations that differ
in every size and option, random model folders in temporary places, and the
plain implementation's logits for them."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:  # noqa: BLE001
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device here")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# tiny-llama-A: plain rotary, tied head, 2 query heads per key/value head.
TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0,
    "rope_scaling": None, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
    "max_position_embeddings": 1024, "eos_token_id": 2,
}
# tiny-llama-B: llama3-scaled rotary, separate head, 3 query heads on 1 key/value
# head, sizes that are no power of two, head_dim * heads != hidden.
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
    "head_dim": 48, "intermediate_size": 264, "vocab_size": 391, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 32},
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 2048,
    "eos_token_id": [5, 7],
}
TINY = {"A": TINY_A, "B": TINY_B}
# The two tiny configurations exactly as the benchmark description words them (the
# ones above are harder variants: a head size of 48, sizes that are no multiple of
# 8, larger weights).  (configuration, seed, std of matrices, std of norm scales,
# prompt lengths, decode steps, temperature, sampling seed)
NAMED_TINY = {
    "tiny-llama-A": (dict(TINY_A, max_position_embeddings=128), 0, 0.02, 0.01, (5, 17, 32), 16, 0.0, 0),
    "tiny-llama-B": (dict(TINY_B, head_dim=32, intermediate_size=256, vocab_size=384, max_position_embeddings=256),
                     1, 0.03, 0.02, (1, 9, 40, 64), 24, 0.8, 7),
}
# (seed, std of matrices, std of norm scales around 1).  The stds are far larger
# than a trained model's so that attention is peaked and a wrong key, a wrong
# position or a wrong page changes the logits visibly.
TINY_INIT = {"A": (0, 0.12, 0.05), "B": (1, 0.10, 0.08)}


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """name -> folder with config.json and bfloat16 model.safetensors.  Stored in
    bfloat16 so that the float32 path, the bfloat16 path and the plain
    implementation all see exactly the same weight values."""
    import go_tinygrad_b200 as lib
    out = {}
    for name, cfg in TINY.items():
        seed, std, norm_std = TINY_INIT[name]
        folder = str(tmp_path_factory.mktemp(f"tiny_{name}"))
        lib.write_random_model(folder, cfg, seed=seed, dtype="bfloat16", std=std, norm_std=norm_std)
        out[name] = folder
    return out


@pytest.fixture(scope="session")
def plain_models(model_folders):
    import plain_llama
    return {name: plain_llama.read_model(folder) for name, folder in model_folders.items()}


class PlainLogits:
    """Logits of the plain implementation, computed once per token sequence."""

    def __init__(self, plain_models):
        self._models = plain_models
        self._memo = {}

    def __call__(self, name, tokens):
        import plain_llama
        key = (name, tuple(int(t) for t in tokens))
        if key not in self._memo:
            cfg, w = self._models[name]
            self._memo[key] = plain_llama.forward(cfg, w, list(key[1]))
        return self._memo[key]


@pytest.fixture(scope="session")
def plain_logits(plain_models):
    return PlainLogits(plain_models)


def make_prompts(name, lengths, seed=0):
    rng = np.random.default_rng(seed)
    vocab = TINY[name]["vocab_size"]
    return [rng.integers(0, vocab, n).tolist() for n in lengths]


# Tolerances, fixed once.  float32: the engine and the plain implementation
# differ in summation order only.  bfloat16: activations are rounded to 8 bits
# of mantissa between kernels (weights are identical), and the error is judged
# against the size of the logits.
def assert_close(got, want, dtype, what=""):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    scale = max(1.0, float(np.abs(want).max()))
    err = np.abs(got - want)
    if dtype == "float32":
        limit_max, limit_mean = 5e-5 * scale, 5e-6 * scale
    else:
        limit_max, limit_mean = 5e-2 * scale, 6e-3 * scale
    worst = np.unravel_index(int(err.argmax()), err.shape)
    assert err.max() <= limit_max, (f"{what}: max error {err.max():.3e} > {limit_max:.3e} at {worst} "
                                    f"(got {got[worst]:.5f}, want {want[worst]:.5f})")
    assert err.mean() <= limit_mean, f"{what}: mean error {err.mean():.3e} > {limit_mean:.3e}"
