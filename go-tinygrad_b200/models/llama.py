"""The dense Llama decoder (SmolLM2, Llama 3.x) as a plan of parts.

This file is the only place that knows the architecture: it maps the typed
configuration to part specs and checkpoint tensor names
(model/llama.go:477-494 for the embedding, final norm and head, :599-613 for a
layer's tensors).  Every layer is a pre-norm block of grouped-query attention
with rotary positions and a SwiGLU feed-forward; layers run in order, each with
a cache entry of its own.
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.registry import Architecture, register_architecture
from ..parts.plan import ModelPlan, PartSpec, default_schedule, pre_norm_layer


def llama_plan(cfg: LlamaConfig) -> ModelPlan:
    rotary = PartSpec("rotary", {
        "head_dim": cfg.head_dim,
        "theta": cfg.rope_theta,
        "scaling": cfg.rope_scaling.to_json() if cfg.rope_scaling else None,
    })
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(pre_norm_layer(
            mixer_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps,
                                            "weight": p + "input_layernorm.weight"}),
            mixer=PartSpec("gqa_attention", {
                "hidden_size": cfg.hidden_size, "n_heads": cfg.num_attention_heads,
                "n_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                "window": None, "scale": None, "position": rotary,
                "q": p + "self_attn.q_proj.weight", "k": p + "self_attn.k_proj.weight",
                "v": p + "self_attn.v_proj.weight", "o": p + "self_attn.o_proj.weight"}),
            feed_forward_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps,
                                                   "weight": p + "post_attention_layernorm.weight"}),
            feed_forward=PartSpec("swiglu", {
                "hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size,
                "gate": p + "mlp.gate_proj.weight", "up": p + "mlp.up_proj.weight",
                "down": p + "mlp.down_proj.weight"}),
        ))
    embed_name = "model.embed_tokens.weight"
    if cfg.tie_word_embeddings:
        head = PartSpec("lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                    "weight": embed_name, "tied": True, "ignored": "lm_head.weight"})
    else:
        head = PartSpec("lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                    "weight": "lm_head.weight"})
    plan = ModelPlan(
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size,
                                               "hidden_size": cfg.hidden_size, "weight": embed_name}),
        layers=tuple(layers),
        schedule=default_schedule(cfg.num_hidden_layers),
        final_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps,
                                        "weight": "model.norm.weight"}),
        head=head,
        stop_tokens=tuple(cfg.eos_token_ids),
        max_position=cfg.max_position_embeddings,
    )
    plan.check()
    return plan


LLAMA = register_architecture(Architecture(
    names=("LlamaForCausalLM", "llama"),
    read_config=LlamaConfig.from_json,
    plan=llama_plan,
    # older exporters store each layer's rotary frequencies as a buffer; they are
    # recomputed from the configuration here and the stored copy is not read
    ignore=("*.rotary_emb.inv_freq",),
))
