"""Configuration, registry, safetensors container and weight binding (no GPU)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

import go_tinygrad_b200 as lib
from go_tinygrad_b200.config import (Architecture, ConfigError, LlamaConfig, find_architecture,
                                     read_model_config, register_architecture,
                                     unregister_architecture)
from go_tinygrad_b200.parts import plan_weight_specs
from go_tinygrad_b200.weights import (SafetensorsError, SafetensorsFile, TensorSource, WeightError,
                                      bind, write_safetensors)
from conftest import TINY_A, TINY_B


# ------------------------------------------------------------------- configuration
def test_defaults_and_derived_sizes():
    cfg = LlamaConfig.from_json({"vocab_size": 100, "hidden_size": 48, "intermediate_size": 96,
                                 "num_hidden_layers": 2, "num_attention_heads": 6})
    assert cfg.num_key_value_heads == 6 and cfg.head_dim == 8          # model/llama.go:235-237
    assert cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 10000.0      # model/llama.go:223-225
    assert cfg.rope_scaling is None and cfg.tie_word_embeddings is False
    assert (cfg.q_dim, cfg.kv_dim, cfg.group_size) == (48, 48, 1)
    b = LlamaConfig.from_json(TINY_B)
    assert (b.q_dim, b.kv_dim, b.group_size, b.head_dim) == (144, 48, 3, 48)
    assert b.rope_scaling.factor == 8.0 and b.rope_scaling.original_max_position_embeddings == 32
    assert b.eos_token_ids == (5, 7) and LlamaConfig.from_json(TINY_A).eos_token_ids == (2,)


def test_config_round_trip():
    for raw in (TINY_A, TINY_B):
        cfg = LlamaConfig.from_json(raw)
        assert LlamaConfig.from_json(cfg.to_json()) == cfg


@pytest.mark.parametrize("change,match", [
    ({"hidden_size": None}, "hidden_size"),
    ({"vocab_size": 0}, "vocab_size"),
    ({"num_hidden_layers": -1}, "num_hidden_layers"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"hidden_act": "gelu_pytorch_tanh"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0}}, "lacks"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 4.0,
                       "high_freq_factor": 1.0, "original_max_position_embeddings": 32}}, "exceed"),
    ({"rms_norm_eps": -1.0}, "rms_norm_eps"),
    ({"eos_token_id": "x"}, "eos_token_id"),
])
def test_config_errors(change, match):
    raw = dict(TINY_A)
    for k, v in change.items():
        if v is None:
            raw.pop(k)
        else:
            raw[k] = v
    with pytest.raises(ConfigError, match=match):
        LlamaConfig.from_json(raw)


def test_registry_lookup_and_unknown(tmp_path):
    assert find_architecture({"architectures": ["LlamaForCausalLM"]}) is find_architecture({"model_type": "llama"})
    with pytest.raises(ConfigError, match="registered"):
        find_architecture({"architectures": ["Qwen3MoeForCausalLM"], "model_type": "qwen3_moe"})
    with pytest.raises(ConfigError, match="neither"):
        find_architecture({})
    with pytest.raises(ConfigError, match="does not exist"):
        read_model_config(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    arch, cfg = read_model_config(str(tmp_path))
    assert "llama" in arch.names and cfg.hidden_size == 96
    toy = Architecture(("ToyForCausalLM",), LlamaConfig.from_json, arch.plan)
    register_architecture(toy)
    try:
        assert find_architecture({"architectures": ["ToyForCausalLM"]}) is toy
        with pytest.raises(ValueError, match="already registered"):
            register_architecture(Architecture(("ToyForCausalLM",), LlamaConfig.from_json, arch.plan))
    finally:
        unregister_architecture(toy)


def test_the_plan_carries_every_size_from_the_configuration():
    for raw in (TINY_A, TINY_B):
        cfg = LlamaConfig.from_json(raw)
        plan = find_architecture(raw).plan(cfg)
        assert len(plan.layers) == cfg.num_hidden_layers == len(plan.schedule)
        specs = {s.name: s for s in plan_weight_specs(plan)}
        assert specs["model.embed_tokens.weight"].shape == (cfg.vocab_size, cfg.hidden_size)
        assert specs["model.layers.0.self_attn.q_proj.weight"].shape == (cfg.q_dim, cfg.hidden_size)
        assert specs["model.layers.1.self_attn.k_proj.weight"].shape == (cfg.kv_dim, cfg.hidden_size)
        assert specs["model.layers.1.self_attn.o_proj.weight"].shape == (cfg.hidden_size, cfg.q_dim)
        assert specs["model.layers.0.mlp.down_proj.weight"].shape == (cfg.hidden_size, cfg.intermediate_size)
        assert specs["model.norm.weight"].role == "vector"
        assert ("lm_head.weight" in specs and not specs["lm_head.weight"].optional) != cfg.tie_word_embeddings
        assert plan.stop_tokens == cfg.eos_token_ids


# --------------------------------------------------------------------- safetensors
def test_safetensors_round_trip(tmp_path):
    tensors = {"a": torch.arange(6, dtype=torch.float32).reshape(2, 3),
               "b": torch.tensor([1.5, -2.25], dtype=torch.bfloat16),
               "c": torch.tensor([[1.0, 2.0]], dtype=torch.float16),
               "table": torch.tensor([3, 1 << 20], dtype=torch.int64),
               "i": torch.tensor([7], dtype=torch.int32)}
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, tensors)
    f = SafetensorsFile(path)
    assert sorted(f.names()) == sorted(tensors)
    for name, t in tensors.items():
        got = f.tensor(name)
        if t.dtype == torch.int64:
            assert got.dtype == torch.int32 and got.tolist() == t.tolist()     # integer tables as int32
        else:
            assert got.dtype == t.dtype and torch.equal(got, t)                # stored dtype is kept
    f.close()


def _raw_file(path, header, data=b""):
    head = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)) + head + data)


def test_safetensors_malformed(tmp_path):
    p = str(tmp_path / "model.safetensors")
    with open(p, "wb") as f:
        f.write(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(p)
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(p)
    # the three cases of loader/safetensors/safetensors_test.go:140-159
    _raw_file(p, {"x": {"dtype": "F32", "shape": [2], "data_offsets": [4, 2]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="offsets"):
        SafetensorsFile(p)
    _raw_file(p, {"x": {"dtype": "F32", "shape": [2], "data_offsets": [0, 16]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="offsets"):
        SafetensorsFile(p)
    _raw_file(p, {"x": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="needs 12 bytes"):
        SafetensorsFile(p)
    _raw_file(p, {"x": {"dtype": "F8_E4M3", "shape": [8], "data_offsets": [0, 8]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        SafetensorsFile(p)
    with pytest.raises(FileNotFoundError):
        TensorSource(str(tmp_path / "nowhere"))


def test_sharded_folder(tmp_path):
    write_safetensors(str(tmp_path / "s1.safetensors"), {"a": torch.ones(2)})
    write_safetensors(str(tmp_path / "s2.safetensors"), {"b": torch.zeros(3)})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    with TensorSource(str(tmp_path)) as src:
        assert sorted(src.names()) == ["a", "b"] and src.tensor("b").shape == (3,)
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "s1.safetensors", "b": "gone.safetensors"}}))
    with pytest.raises(SafetensorsError, match="missing"):
        TensorSource(str(tmp_path))


# ------------------------------------------------------------------------- binding
def test_random_model_folder_and_binding(tmp_path):
    folder = str(tmp_path / "m")
    lib.write_random_model(folder, TINY_B, seed=3, dtype="bfloat16", std=0.05, norm_std=0.02)
    arch, cfg = read_model_config(folder)
    specs = plan_weight_specs(arch.plan(cfg))
    with TensorSource(folder) as src:
        tensors = bind(src, specs)
    assert set(tensors) == {s.name for s in specs if not s.optional}
    q = tensors["model.layers.2.self_attn.q_proj.weight"]
    assert q.dtype == torch.bfloat16 and q.shape == (144, 96)
    assert abs(float(q.float().std()) - 0.05) < 0.005
    n = tensors["model.norm.weight"].float()
    assert abs(float(n.mean()) - 1.0) < 0.01 and 0.01 < float(n.std()) < 0.03
    # the same seed writes the same bytes; another seed does not
    again, other = str(tmp_path / "again"), str(tmp_path / "other")
    lib.write_random_model(again, TINY_B, seed=3, dtype="bfloat16", std=0.05, norm_std=0.02)
    lib.write_random_model(other, TINY_B, seed=4, dtype="bfloat16", std=0.05, norm_std=0.02)
    read = lambda d: open(os.path.join(d, "model.safetensors"), "rb").read()
    assert read(folder) == read(again) != read(other)
    # a float32 folder keeps 32-bit tensors 32-bit
    f32 = str(tmp_path / "f32")
    lib.write_random_model(f32, TINY_A, seed=0, dtype="float32")
    with TensorSource(f32) as src:
        assert src.tensor("model.layers.0.mlp.up_proj.weight").dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = str(tmp_path / "m")
    lib.write_random_model(folder, TINY_A, seed=0, dtype="bfloat16")
    path = os.path.join(folder, "model.safetensors")
    with TensorSource(folder) as src:
        tensors = {n: src.tensor(n) for n in src.names()}
    del tensors["model.layers.1.mlp.gate_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.2.self_attn.q_proj.weight"] = torch.zeros(64, 64)      # a layer too many
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64)      # wrong shape
    tensors["model.layers.0.input_layernorm.weight"] = torch.zeros(64, dtype=torch.int32)
    write_safetensors(path, tensors)
    arch, cfg = read_model_config(folder)
    with TensorSource(folder) as src, pytest.raises(WeightError) as err:
        bind(src, plan_weight_specs(arch.plan(cfg)))
    e = err.value
    assert e.missing == ["model.layers.1.mlp.gate_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.2.self_attn.q_proj.weight"]
    assert e.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (32, 64), (16, 64))]
    assert e.wrong_dtype == [("model.layers.0.input_layernorm.weight", "torch.int32")]
    text = str(e)
    for needle in ("missing (2)", "unexpected (1)", "is [16, 64], the model needs [32, 64]", "gate_proj"):
        assert needle in text


def test_tied_head_tolerates_a_stray_lm_head_and_untied_needs_one(tmp_path):
    folder = str(tmp_path / "m")
    lib.write_random_model(folder, TINY_A, seed=0, dtype="bfloat16")
    path = os.path.join(folder, "model.safetensors")
    with TensorSource(folder) as src:
        tensors = {n: src.tensor(n) for n in src.names()}
    assert "lm_head.weight" not in tensors
    tensors["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)
    write_safetensors(path, tensors)
    arch, cfg = read_model_config(folder)
    with TensorSource(folder) as src:
        assert "lm_head.weight" not in bind(src, plan_weight_specs(arch.plan(cfg)))
    folder_b = str(tmp_path / "b")
    lib.write_random_model(folder_b, TINY_B, seed=0, dtype="bfloat16")
    with TensorSource(folder_b) as src:
        tensors = {n: src.tensor(n) for n in src.names()}
    del tensors["lm_head.weight"]
    write_safetensors(os.path.join(folder_b, "model.safetensors"), tensors)
    arch, cfg = read_model_config(folder_b)
    with TensorSource(folder_b) as src, pytest.raises(WeightError, match="lm_head.weight"):
        bind(src, plan_weight_specs(arch.plan(cfg)))


def test_buffers_an_architecture_names_are_passed_over_and_nothing_else(tmp_path):
    """Older exporters of this architecture store each layer's rotary frequencies
    (self_attn.rotary_emb.inv_freq).  The architecture's registry entry names that
    pattern; such tensors are not read and are no error, while any other tensor
    nobody declared still is, and a view handed out without a copy reads the same
    bytes as a copy."""
    folder = str(tmp_path / "m")
    lib.write_random_model(folder, TINY_A, seed=0, dtype="bfloat16")
    path = os.path.join(folder, "model.safetensors")
    with TensorSource(folder) as src:
        tensors = {n: src.tensor(n) for n in src.names()}
    for layer in range(2):
        tensors[f"model.layers.{layer}.self_attn.rotary_emb.inv_freq"] = torch.ones(8)
    write_safetensors(path, tensors)
    arch, cfg = read_model_config(folder)
    assert "*.rotary_emb.inv_freq" in arch.ignore
    specs = plan_weight_specs(arch.plan(cfg))
    with TensorSource(folder) as src, pytest.raises(WeightError) as err:
        bind(src, specs)                                   # without the architecture's patterns: unexpected
    assert len(err.value.unexpected) == 2
    with TensorSource(folder) as src:
        bound = bind(src, specs, ignore=arch.ignore)
        views = bind(src, specs, ignore=arch.ignore, copy=False)
        assert not any("inv_freq" in n for n in bound) and set(views) == set(bound)
        for n in bound:
            assert torch.equal(bound[n], views[n]) and bound[n].dtype == torch.bfloat16
        del views
    tensors["model.layers.0.self_attn.rotary_emb.cos_cached"] = torch.ones(8)
    write_safetensors(path, tensors)
    with TensorSource(folder) as src, pytest.raises(WeightError) as err:
        bind(src, specs, ignore=arch.ignore)
    assert err.value.unexpected == ["model.layers.0.self_attn.rotary_emb.cos_cached"]
