"""What every part of a model is: registries, the run's settings, and the
per-step context parts receive.

Categories: ``embedding``, ``norm``, ``position``, ``mixer``, ``feed_forward``,
``block`` and ``head``.  A part is registered under (category, kind) and built
from a `PartSpec`; it declares its tensors (`weight_specs`), takes them
(`load`) and computes (`forward`, whose signature its category fixes -- see the
category base classes below).  Adding a part is registering a class; nothing in
the engine names a kind.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Mapping, Optional, Tuple, Type

import torch

from ..cache import CacheHandle, Request
from ..kernels import ops
from ..weights.binder import WeightSpec
from .plan import PartSpec

CATEGORIES = ("embedding", "norm", "position", "mixer", "feed_forward", "block", "head")
_REGISTRY: Dict[Tuple[str, str], Type["Part"]] = {}


def register_part(category: str, kind: str, replace: bool = False):
    """Class decorator: make `kind` available to plans under `category`."""
    if category not in CATEGORIES:
        raise ValueError(f"unknown part category {category!r}; categories: {CATEGORIES}")

    def deco(cls):
        if (category, kind) in _REGISTRY and not replace and _REGISTRY[(category, kind)] is not cls:
            raise ValueError(f"{category} part {kind!r} is already registered")
        _REGISTRY[(category, kind)] = cls
        cls.category, cls.kind = category, kind
        return cls
    return deco


def unregister_part(category: str, kind: str) -> None:
    _REGISTRY.pop((category, kind), None)


def registered_parts(category: Optional[str] = None) -> List[Tuple[str, str]]:
    return sorted(k for k in _REGISTRY if category is None or k[0] == category)


def build_part(category: str, spec: PartSpec) -> "Part":
    cls = _REGISTRY.get((category, spec.kind))
    if cls is None:
        known = [k for c, k in registered_parts(category)]
        raise KeyError(f"no {category} part of kind {spec.kind!r} is registered; registered: {known}")
    return cls(spec)


@dataclass
class Runtime:
    """Settings of a run that parts need: where tensors live and the compute
    dtype (torch.bfloat16: the serving kernels; torch.float32: everything in
    true 32-bit)."""
    device: torch.device
    dtype: torch.dtype
    _shared: Dict[str, torch.Tensor] = field(default_factory=dict, repr=False)

    def matrix(self, t: torch.Tensor, share_as: Optional[str] = None) -> torch.Tensor:
        """A weight matrix or table on the device in the compute dtype.  Parts
        that pass the same `share_as` (the tensor's checkpoint name) get one
        device copy: a tied head and the embedding share their table this way."""
        if share_as is not None and share_as in self._shared:
            return self._shared[share_as]
        out = t.to(device=self.device, dtype=self.dtype).contiguous()
        if share_as is not None:
            self._shared[share_as] = out
        return out

    def vector(self, t: torch.Tensor) -> torch.Tensor:
        """A scale vector on the device, always float32."""
        return t.to(device=self.device, dtype=torch.float32).contiguous()

    def empty(self, *shape: int, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)


@dataclass
class StepContext:
    """One step's batch as the parts see it.  Tokens of all sequences are packed
    in one row dimension of length `n_tokens`; sequence b owns rows
    cu_seqlens[b]..cu_seqlens[b+1] at positions start_pos[b], start_pos[b]+1, ...
    Device tensors are int32."""
    rt: Runtime
    n_tokens: int
    n_seqs: int
    tokens: torch.Tensor        # [n_tokens]
    positions: torch.Tensor     # [n_tokens] absolute position of each token
    token_seq: torch.Tensor     # [n_tokens] index of the token's sequence in the batch
    cu_seqlens: torch.Tensor    # [n_seqs + 1]
    slots: torch.Tensor         # [n_seqs] cache slot of each sequence
    start_pos: torch.Tensor     # [n_seqs] tokens already in the cache before this step
    max_q_len: int              # longest run of new tokens in the batch
    max_kv_len: int             # longest sequence after this step
    is_decode: bool             # every sequence brings exactly one token
    shared: Dict[Any, Any] = field(default_factory=dict)   # per-step values parts share (rotary tables)
    update_into: Optional["ResidualStream"] = None   # set by a block around a part's forward: see emit_update


class Part:
    category: str = ""
    kind: str = ""

    def __init__(self, spec: PartSpec):
        self.spec = spec
        self.p: Mapping[str, Any] = spec.params

    def weight_specs(self) -> List[WeightSpec]:
        return []

    def load(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        """Take the declared tensors (host, stored dtype) and keep what `forward` needs."""

    def param(self, name: str, default: Any = None) -> Any:
        if name in self.p:
            return self.p[name]
        if default is not None:
            return default
        raise KeyError(f"{self.category} part {self.kind!r} needs parameter {name!r}")


class ResidualStream:
    """The hidden state between parts: a float32 `residual` [N, H] and a
    `pending` update in the compute dtype that has not been added yet.  A norm
    adds the pending update and normalises in one pass."""

    def __init__(self, residual: torch.Tensor, pending: Optional[torch.Tensor] = None):
        self.residual = residual
        self.pending = pending


def emit_update(x: torch.Tensor, w: torch.Tensor, ctx: "StepContext") -> Optional[torch.Tensor]:
    """The last product of a mixer or feed-forward: its update x . w^T, [n_tokens, H].
    When the block has offered its residual stream (`ctx.update_into`) and the
    product can add to it in its epilogue (a prompt step in bfloat16), the update
    is added there and None is returned in its place: it never goes through
    memory, and the norm that follows has nothing left to add."""
    stream = ctx.update_into
    if (stream is not None and stream.pending is None and ctx.rt.dtype == torch.bfloat16
            and ops.linear_add_residual(x, w, stream.residual)):
        return None
    out = ctx.rt.empty(x.shape[0], w.shape[0])
    ops.linear(x, w, out)
    return out


# ---- category interfaces --------------------------------------------------------
class Embedding(Part):
    def forward(self, ctx: StepContext) -> ResidualStream:
        raise NotImplementedError


class Norm(Part):
    def forward(self, stream: ResidualStream, ctx: StepContext,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Add the pending update into the residual, return the normalised rows
        (all, or the int32 row indices `rows`) in the compute dtype."""
        raise NotImplementedError


class PositionEncoding(Part):
    def on_embedding(self, stream: ResidualStream, ctx: StepContext) -> None:
        """Hook for encodings that act on the embedded tokens (absolute positions)."""

    def rotation(self, ctx: StepContext) -> Optional[torch.Tensor]:
        """For rotary encodings: float32 [n_tokens, head_dim/2, 2] of (cos, sin) for
        this step's tokens, or None for no rotation of queries and keys."""
        return None


class Mixer(Part):
    def cache_requests(self) -> List[Request]:
        return []

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheHandle) -> torch.Tensor:
        """x: normalised [n_tokens, H] in the compute dtype -> update [n_tokens, H]."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """An arrangement of a mixer and a feed-forward with their norms."""

    def assemble(self, mixer_norm: Norm, mixer: Mixer, ff_norm: Norm, ff: FeedForward) -> None:
        self.mixer_norm, self.mixer, self.ff_norm, self.ff = mixer_norm, mixer, ff_norm, ff

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: CacheHandle) -> None:
        raise NotImplementedError


class Head(Part):
    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        """x: normalised wanted rows [R, H] -> float32 logits [R, V]."""
        raise NotImplementedError
