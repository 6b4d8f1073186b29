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


class _Region:
    """One stretch of a workspace: tensors are cut from a buffer front to back;
    `reset` makes the whole buffer free again, grown to what the last round asked
    for.  What does not fit is a tensor of its own."""
    ALIGN = 256

    def __init__(self, device: torch.device):
        self.device = device
        self.buffer: Optional[torch.Tensor] = None
        self.offset = 0
        self.asked = 0                      # bytes asked for since the last reset

    def reset(self) -> None:
        if self.asked > (self.buffer.numel() if self.buffer is not None else 0) and not self._recording():
            # a quarter more than was asked for: the sizes of a step's scratch vary a little
            self.buffer = torch.empty(self.asked + self.asked // 4, dtype=torch.uint8, device=self.device)
        self.offset = self.asked = 0

    def _recording(self) -> bool:
        """While a CUDA graph is being recorded the buffer is not replaced: memory
        allocated then belongs to the recording."""
        return self.device.type == "cuda" and torch.cuda.is_current_stream_capturing()

    def take(self, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = n * dtype.itemsize
        padded = (nbytes + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        self.asked += padded
        if self.buffer is None or self.offset + padded > self.buffer.numel():
            return torch.empty(shape, dtype=dtype, device=self.device)
        out = self.buffer[self.offset:self.offset + nbytes].view(dtype).view(shape)
        self.offset += padded
        return out


class Workspace:
    """Where the intermediate tensors of a step live, so that a step of a size
    that has run before asks the allocator for nothing.  Three regions: one for
    what lasts the whole step (the residual stream, the step's metadata, tables)
    and two that take turns layer by layer -- what a layer allocates stays valid
    until the layer after it has ended, which is as long as an update left
    pending on the residual stream needs.  The engine calls `begin_step` and
    `next_layer`; without those calls nothing is ever handed out twice.  A step
    of a new size finds the regions too small, gets ordinary tensors for the
    rest, and the regions grow at their next reset.  A buffer that is replaced
    lives on for as long as a tensor (or a recorded graph's owner) holds it."""

    def __init__(self, device: torch.device):
        self.step_region = _Region(device)
        self.layer_regions = (_Region(device), _Region(device))
        self.turn = 0

    def begin_step(self) -> None:
        self.step_region.reset()
        for r in self.layer_regions:
            r.reset()
        self.turn = 0

    def next_layer(self) -> None:
        self.turn ^= 1
        self.layer_regions[self.turn].reset()

    def take(self, shape: Tuple[int, ...], dtype: torch.dtype, lifetime: str) -> torch.Tensor:
        if lifetime == "step":
            return self.step_region.take(shape, dtype)
        if lifetime != "layer":
            raise ValueError(f"a workspace tensor lasts a 'layer' or a 'step', not {lifetime!r}")
        return self.layer_regions[self.turn].take(shape, dtype)

    def buffers(self) -> List[torch.Tensor]:
        """The buffers in use now (held by whoever records a graph over them)."""
        return [r.buffer for r in (self.step_region,) + self.layer_regions if r.buffer is not None]


@dataclass
class Runtime:
    """Settings of a run that parts need: where tensors live and the compute
    dtype (torch.bfloat16: the serving kernels; torch.float32: everything in
    true 32-bit)."""
    device: torch.device
    dtype: torch.dtype
    # debugging: every kernel that reads the cache through the block table is preceded by a
    # pass that checks the same indices on the device (ops.checked_access); steps then
    # synchronise and are not recorded as graphs
    check_access: bool = False
    _shared: Dict[str, torch.Tensor] = field(default_factory=dict, repr=False)
    _workspace: Optional[Workspace] = field(default=None, repr=False)

    @property
    def workspace(self) -> Workspace:
        if self._workspace is None:
            self._workspace = Workspace(torch.device(self.device))
        return self._workspace

    def matrix(self, t: torch.Tensor, share_as: Optional[str] = None) -> torch.Tensor:
        """A weight matrix or table on the device in the compute dtype.  Parts
        that pass the same `share_as` (the tensor's checkpoint name) get one
        device copy: a tied head and the embedding share their table this way."""
        if share_as is not None and share_as in self._shared:
            return self._shared[share_as]
        out = t.to(device=self.device, dtype=self.dtype).contiguous()
        if out.data_ptr() == t.data_ptr():
            out = out.clone()               # never keep the loader's own memory (it may be a mapped file)
        if share_as is not None:
            self._shared[share_as] = out
        return out

    def vector(self, t: torch.Tensor) -> torch.Tensor:
        """A scale vector on the device, always float32."""
        out = t.to(device=self.device, dtype=torch.float32).contiguous()
        return out.clone() if out.data_ptr() == t.data_ptr() else out

    def empty(self, *shape: int, dtype: Optional[torch.dtype] = None, lifetime: str = "layer") -> torch.Tensor:
        """An uninitialised intermediate of the running step, from the workspace:
        valid until the layer after the one that asked has ended (lifetime
        "layer") or until the step ends ("step").  Nothing from here may be kept
        across steps; what is handed to the caller of the step comes from `result`."""
        return self.workspace.take(tuple(int(d) for d in shape), dtype or self.dtype, lifetime)

    def result(self, *shape: int, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """An uninitialised tensor of its own, for what outlives the step."""
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
    total_kv_len: int = 0       # all sequences' lengths after this step, added up (0: not known)
    shared: Dict[Any, Any] = field(default_factory=dict)   # per-step values parts share (rotary tables)
    update_into: Optional["ResidualStream"] = None   # set by a block around a part's forward: see emit_update
    step: int = 0               # which step of the model this is (counted by the model; for `op_hook`)
    layer: int = -1             # the layer that is running (set by the engine before each block)
    op_hook: Optional[Callable[[int, int, str, torch.Tensor], None]] = None

    def trace(self, op: str, tensor) -> None:
        """Hand a named intermediate value of the running layer to the hook, if one
        is set: `op_hook(step, layer, op, tensor)`.  `tensor` may be a function
        that builds the value, called only when a hook listens.  The names follow
        the reference's per-op hook (model/debug_hooks.go:5-7 and its call sites in
        model/llama.go:1089-1427): hidden_in, normed, q, k, v, q_attn, attn, o,
        mlp_input, gate_pre, up, gate_act, down, hidden_post_ffn.  A part reports
        what it materialises: a fused kernel that never writes a value to memory
        has nothing to report under that name."""
        if self.op_hook is not None:
            self.op_hook(self.step, self.layer, op, tensor() if callable(tensor) else tensor)


class Part:
    category: str = ""
    kind: str = ""
    # False for a part whose forward talks to the host (reads a device value, picks
    # rows by data): a step that contains it cannot be recorded as a CUDA graph,
    # and the generation loop then launches its decode steps kernel by kernel.
    capturable: bool = True

    def __init__(self, spec: PartSpec):
        self.spec = spec
        self.p: Mapping[str, Any] = spec.params

    def children(self) -> List["Part"]:
        """Parts this part built from nested specs and owns (a mixer's position
        encoding, a block's norms, mixer and feed-forward).  The model walks them:
        their tensors are declared, bound and loaded with everyone else's."""
        return []

    def weight_specs(self) -> List[WeightSpec]:
        """The tensors of this part itself (its children declare their own)."""
        return []

    def load(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        """Take the declared tensors (host, stored dtype) and keep what `forward` needs."""

    def param(self, name: str, default: Any = None) -> Any:
        if name in self.p:
            return self.p[name]
        if default is not None:
            return default
        raise KeyError(f"{self.category} part {self.kind!r} needs parameter {name!r}")


def walk(part: "Part"):
    """`part`, then everything below it, parents before children."""
    yield part
    for child in part.children():
        yield from walk(child)


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
    # How a rotary kind pairs the channels of a head and how many it rotates; the
    # kernels that rotate read these.  "half": channel i with i + rotary_dim/2
    # (model/llama.go:1581-1586); "interleaved": 2i with 2i+1.  rotary_dim None:
    # the whole head; otherwise the first `rotary_dim` channels, the rest pass.
    pairing: str = "half"
    rotary_dim: Optional[int] = None

    def on_embedding(self, stream: ResidualStream, ctx: StepContext) -> None:
        """Hook for encodings that act on the embedded tokens (absolute positions)."""

    def rotation(self, ctx: StepContext) -> Optional[torch.Tensor]:
        """For rotary encodings: float32 [n_tokens, rotated channels / 2, 2] of (cos, sin)
        for this step's tokens, or None for no rotation of queries and keys."""
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
    """An arrangement: one layer.  A block kind declares what it is made of in
    `sub_parts`, pairs of (name, category); each is built from the nested
    PartSpec of that name among the block's parameters and becomes an attribute
    of that name.  The block owns them: the model asks the block, never the
    plan, for the parts of a layer, their tensors and their cache needs.  A
    block may declare tensors of its own too (`weight_specs`, `load`)."""
    sub_parts: Tuple[Tuple[str, str], ...] = ()

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        for name, category in self.sub_parts:
            setattr(self, name, build_part(category, self.param(name)))

    def children(self) -> List[Part]:
        return [getattr(self, name) for name, _ in self.sub_parts]

    def cache_requests(self) -> List[Request]:
        """What one run of this layer keeps per sequence: what its parts ask for."""
        requests: List[Request] = []
        for part in walk(self):
            if part is not self and hasattr(part, "cache_requests"):
                requests += part.cache_requests()
        return requests

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: CacheHandle) -> None:
        raise NotImplementedError


class Head(Part):
    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        """x: normalised wanted rows [R, H] -> float32 logits [R, V]."""
        raise NotImplementedError
