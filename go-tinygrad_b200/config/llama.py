"""Typed configuration of the dense Llama decoder (SmolLM2, Llama 3.x).

Every size and constant comes from the keys of the architecture's own
``config.json``; nothing here names a model size.  The keys and their defaults
follow the reference's struct (model/llama.go:36-49) and its normalisation
(model/llama.go:223-237: rms_norm_eps 0 -> 1e-5, head_dim 0 -> hidden/heads).
The ``rope_scaling`` block (llama3 frequency scaling) is not read by the
reference at all; it is parsed here because Llama 3.x checkpoints carry it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


class ConfigError(ValueError):
    """config.json is missing a key, or a value is out of range."""


@dataclass(frozen=True)
class RopeScaling:
    """The llama3 frequency-scaling block of ``rope_scaling``."""
    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    @staticmethod
    def from_json(block: Optional[Mapping[str, Any]]) -> Optional["RopeScaling"]:
        if block is None:
            return None
        if not isinstance(block, Mapping):
            raise ConfigError("rope_scaling must be an object or null")
        kind = block.get("rope_type", block.get("type"))
        if kind in (None, "default"):
            return None
        if kind != "llama3":
            raise ConfigError(f"rope_scaling type {kind!r} is not supported (supported: 'llama3')")
        need = ("factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings")
        missing = [k for k in need if k not in block]
        if missing:
            raise ConfigError(f"rope_scaling (llama3) lacks {missing}")
        rs = RopeScaling("llama3", float(block["factor"]), float(block["low_freq_factor"]),
                         float(block["high_freq_factor"]),
                         int(block["original_max_position_embeddings"]))
        if rs.factor <= 0 or rs.original_max_position_embeddings <= 0:
            raise ConfigError("rope_scaling: factor and original_max_position_embeddings must be positive")
        if not rs.high_freq_factor > rs.low_freq_factor:
            raise ConfigError("rope_scaling: high_freq_factor must exceed low_freq_factor")
        return rs

    def to_json(self) -> dict:
        return {"rope_type": self.rope_type, "factor": self.factor,
                "low_freq_factor": self.low_freq_factor,
                "high_freq_factor": self.high_freq_factor,
                "original_max_position_embeddings": self.original_max_position_embeddings}


def _positive_int(raw: Mapping[str, Any], key: str, default: Optional[int] = None) -> int:
    v = raw.get(key, None)
    if v is None or v == 0:
        if default is None:
            raise ConfigError(f"config.json lacks {key!r}")
        return default
    if isinstance(v, bool) or not isinstance(v, int) or v < 0:
        raise ConfigError(f"{key!r} must be a positive integer, got {v!r}")
    return v


@dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    rms_norm_eps: float
    tie_word_embeddings: bool
    hidden_act: str = "silu"
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    model_type: str = "llama"
    architectures: Tuple[str, ...] = ("LlamaForCausalLM",)
    torch_dtype: Optional[str] = None
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    # derived sizes ---------------------------------------------------------
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    # reading ---------------------------------------------------------------
    @staticmethod
    def from_json(raw: Mapping[str, Any]) -> "LlamaConfig":
        if not isinstance(raw, Mapping):
            raise ConfigError("config.json must hold an object")
        hidden = _positive_int(raw, "hidden_size")
        heads = _positive_int(raw, "num_attention_heads")
        kv_heads = _positive_int(raw, "num_key_value_heads", default=heads)
        head_dim = _positive_int(raw, "head_dim", default=hidden // heads)
        if head_dim <= 0:
            raise ConfigError("head_dim is 0: hidden_size is smaller than num_attention_heads")
        if heads % kv_heads != 0:
            raise ConfigError(f"num_attention_heads {heads} is not a multiple of "
                              f"num_key_value_heads {kv_heads}")
        if head_dim % 2 != 0:
            raise ConfigError(f"head_dim {head_dim} must be even (rotary pairs)")
        eps = raw.get("rms_norm_eps") or 1e-5
        theta = raw.get("rope_theta") or 10000.0
        if not (isinstance(eps, (int, float)) and eps > 0):
            raise ConfigError(f"rms_norm_eps must be positive, got {eps!r}")
        if not (isinstance(theta, (int, float)) and theta > 0):
            raise ConfigError(f"rope_theta must be positive, got {theta!r}")
        act = raw.get("hidden_act") or raw.get("hidden_activation") or "silu"
        if act != "silu":
            raise ConfigError(f"hidden_act {act!r} is not supported by this architecture (supported: 'silu')")
        for key in ("attention_bias", "mlp_bias"):
            if raw.get(key):
                raise ConfigError(f"{key}=true is not supported (the architecture has no biases)")
        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"eos_token_id must be an integer or a list of integers, got {eos!r}")
        bos = raw.get("bos_token_id")
        if bos is not None and (isinstance(bos, bool) or not isinstance(bos, int)):
            raise ConfigError(f"bos_token_id must be an integer, got {bos!r}")
        archs = raw.get("architectures") or ()
        known = {"vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                 "num_attention_heads", "num_key_value_heads", "head_dim",
                 "max_position_embeddings", "rope_theta", "rope_scaling", "rms_norm_eps",
                 "tie_word_embeddings", "hidden_act", "hidden_activation", "bos_token_id",
                 "eos_token_id", "model_type", "architectures", "torch_dtype",
                 "attention_bias", "mlp_bias"}
        return LlamaConfig(
            vocab_size=_positive_int(raw, "vocab_size"),
            hidden_size=hidden,
            intermediate_size=_positive_int(raw, "intermediate_size"),
            num_hidden_layers=_positive_int(raw, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            max_position_embeddings=_positive_int(raw, "max_position_embeddings", default=2048),
            rope_theta=float(theta),
            rope_scaling=RopeScaling.from_json(raw.get("rope_scaling")),
            rms_norm_eps=float(eps),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            hidden_act=act,
            bos_token_id=bos,
            eos_token_ids=eos_ids,
            model_type=str(raw.get("model_type", "llama")),
            architectures=tuple(str(a) for a in archs),
            torch_dtype=raw.get("torch_dtype"),
            extra={k: v for k, v in raw.items() if k not in known},
        )

    def to_json(self) -> dict:
        """The config.json this configuration is read back from."""
        out = {
            "architectures": list(self.architectures),
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_json() if self.rope_scaling else None,
            "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
        }
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            out["eos_token_id"] = (self.eos_token_ids[0] if len(self.eos_token_ids) == 1
                                   else list(self.eos_token_ids))
        if self.torch_dtype:
            out["torch_dtype"] = self.torch_dtype
        return out
