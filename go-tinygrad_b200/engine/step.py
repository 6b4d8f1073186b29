"""The step function: run the tokens a batch brings, from the cache, and return
logits at the wanted places.

A step takes, for each sequence of the batch, its cache slot, its next tokens
(a whole prompt, or one token, or any run in between) and the places among
these tokens whose logits are wanted.  All tokens of all sequences are packed
into one row dimension -- there is no padding, so padding cannot change a
result -- and every part runs once over the packed rows.  Keys and values are
written for every token; the final norm and the head run on the wanted rows
only.  Afterwards each sequence's length in the cache has grown by its tokens.

The reference runs one token of one sequence per step (the loop body of
model/llama.go:1047-1473) and skips the head for prompt positions before the
last (model/llama.go:1463); its batched prefill (model/batch_prefill.go:20-263)
serves one sequence and quantized weights only.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cache import Cache
from ..kernels import ops
from ..parts.base import ResidualStream, StepContext
from .model import Model


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)   # indices into `tokens`


class StepError(ValueError):
    """The batch handed to `step` is not valid."""


class _Staging:
    """Pinned host buffers the step's metadata is assembled in before its one
    upload.  Two buffers take turns; a buffer is reused only after the copy that
    last read it has completed."""

    def __init__(self, device: torch.device):
        self.device = device
        self.buffers = [None, None]
        self.events = [None, None]
        self.turn = 0

    def upload(self, flat: np.ndarray, rt) -> torch.Tensor:
        n = int(flat.shape[0])
        if self.device.type != "cuda":
            return torch.from_numpy(flat).to(self.device)
        i = self.turn
        self.turn ^= 1
        if self.events[i] is not None:
            self.events[i].synchronize()
        buf = self.buffers[i]
        if buf is None or buf.numel() < n:
            buf = self.buffers[i] = torch.empty(max(4096, 2 * n), dtype=torch.int32, pin_memory=True)
        buf[:n].numpy()[:] = flat
        meta = rt.empty(n, dtype=torch.int32, lifetime="step")
        meta.copy_(buf[:n], non_blocking=True)
        ev = self.events[i] = self.events[i] or torch.cuda.Event()
        ev.record()
        return meta


def _staging(model: Model) -> _Staging:
    st = getattr(model, "_step_staging", None)
    if st is None:
        st = model._step_staging = _Staging(model.rt.device)
    return st


def build_context(model: Model, cache: Cache, entries: Sequence[StepEntry]):
    """Validate the batch, reserve cache pages and upload the step's metadata in
    one copy.  Returns (context, wanted row indices on the device or None)."""
    if not entries:
        raise StepError("a step needs at least one sequence")
    vocab = model.plan.vocab_size
    tok_parts, pos_parts, seq_parts, want_parts = [], [], [], []
    cu = [0]
    slots: List[int] = []
    start: List[int] = []
    seen = set()
    for b, e in enumerate(entries):
        toks = np.asarray(e.tokens, dtype=np.int64).reshape(-1)
        n = int(toks.shape[0])
        if n == 0:
            raise StepError(f"sequence {b} of the batch brings no tokens")
        if e.slot in seen:
            raise StepError(f"slot {e.slot} appears twice in one batch")
        seen.add(e.slot)
        if not cache.slots.is_held(e.slot):
            raise StepError(f"slot {e.slot} is not open")
        if toks.min() < 0 or toks.max() >= vocab:
            bad = toks[(toks < 0) | (toks >= vocab)][0]
            raise StepError(f"token id {int(bad)} is outside the vocabulary of {vocab}")
        s0 = cache.length(e.slot)
        if len(e.want):
            want = np.asarray(e.want, dtype=np.int64).reshape(-1)
            if want.min() < 0 or want.max() >= n:
                bad = want[(want < 0) | (want >= n)][0]
                raise StepError(f"wanted place {int(bad)} is outside the {n} tokens of sequence {b}")
            want_parts.append(want + cu[-1])
        tok_parts.append(toks)
        pos_parts.append(np.arange(s0, s0 + n, dtype=np.int64))
        seq_parts.append(np.full(n, b, dtype=np.int64))
        cu.append(cu[-1] + n)
        slots.append(e.slot)
        start.append(s0)
    cache.reserve_many([(e.slot, s + len(e.tokens)) for e, s in zip(entries, start)])
    cache.flush_tables()

    n_tok, n_seq = cu[-1], len(entries)
    n_want = sum(int(w.shape[0]) for w in want_parts)
    flat = np.concatenate(tok_parts + pos_parts + seq_parts +
                          [np.asarray(cu), np.asarray(slots), np.asarray(start)] + want_parts).astype(np.int32)
    meta = _staging(model).upload(flat, model.rt)
    o = 0

    def take(k):
        nonlocal o
        v = meta[o:o + k]
        o += k
        return v
    ctx = StepContext(
        rt=model.rt, n_tokens=n_tok, n_seqs=n_seq,
        tokens=take(n_tok), positions=take(n_tok), token_seq=take(n_tok),
        cu_seqlens=take(n_seq + 1), slots=take(n_seq), start_pos=take(n_seq),
        max_q_len=max(len(e.tokens) for e in entries),
        max_kv_len=max(s + len(e.tokens) for s, e in zip(start, entries)),
        is_decode=all(len(e.tokens) == 1 for e in entries),
        total_kv_len=sum(s + len(e.tokens) for s, e in zip(start, entries)),
        step=model.steps_run, op_hook=model.op_hook,
    )
    rows = take(n_want) if n_want else None
    return ctx, rows


def run_layers(model: Model, cache: Cache, ctx: StepContext) -> ResidualStream:
    """Embedding, then every schedule entry in order."""
    workspace = model.rt.workspace
    stream = model.embedding.forward(ctx)
    for i, entry in enumerate(model.plan.schedule):
        ctx.layer = entry.layer
        workspace.next_layer()              # what the layer before the last one allocated is free again
        model.blocks[entry.layer].forward(stream, ctx, cache.handles[i])
    ctx.layer = -1
    return stream


def logits_at(model: Model, stream: ResidualStream, ctx: StepContext,
              rows: Optional[torch.Tensor]) -> torch.Tensor:
    """Final norm and head on the wanted rows only: float32 [n_wanted, vocab]."""
    if rows is None:
        return torch.empty((0, model.plan.vocab_size), dtype=torch.float32, device=model.rt.device)
    x = model.final_norm.forward(stream, ctx, rows=rows)
    return model.head.forward(x, ctx)


def step(model: Model, cache: Cache, entries: Sequence[StepEntry]) -> torch.Tensor:
    """Run one step; returns float32 logits [sum of len(want), vocab] on the
    device, in the order of the entries and of each entry's `want`."""
    if not model.loaded:
        raise StepError("the model has no weights loaded")
    model.rt.workspace.begin_step()         # the intermediates of the step before are dead
    ctx, rows = build_context(model, cache, entries)
    # each kernel may set itself up while its predecessor drains (kernels that take
    # no part in this are launched the plain way and order themselves fully)
    with ops.chained_launches(model.rt.device.type == "cuda"), ops.checked_access(model.rt.check_access):
        stream = run_layers(model, cache, ctx)
        logits = logits_at(model, stream, ctx, rows)
    for e in entries:
        cache.advance(e.slot, len(e.tokens))
    model.steps_run += 1
    return logits
