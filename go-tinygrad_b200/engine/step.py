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

import torch

from ..cache import Cache
from ..parts.base import ResidualStream, StepContext
from .model import Model


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)   # indices into `tokens`


class StepError(ValueError):
    """The batch handed to `step` is not valid."""


def build_context(model: Model, cache: Cache, entries: Sequence[StepEntry]):
    """Validate the batch, reserve cache pages and upload the step's metadata in
    one copy.  Returns (context, wanted row indices on the device or None)."""
    if not entries:
        raise StepError("a step needs at least one sequence")
    vocab = model.plan.vocab_size
    tokens: List[int] = []
    positions: List[int] = []
    token_seq: List[int] = []
    cu = [0]
    slots: List[int] = []
    start: List[int] = []
    want_rows: List[int] = []
    seen = set()
    for b, e in enumerate(entries):
        n = len(e.tokens)
        if n == 0:
            raise StepError(f"sequence {b} of the batch brings no tokens")
        if e.slot in seen:
            raise StepError(f"slot {e.slot} appears twice in one batch")
        seen.add(e.slot)
        if not cache.slots.is_held(e.slot):
            raise StepError(f"slot {e.slot} is not open")
        s0 = cache.length(e.slot)
        for t in e.tokens:
            if not 0 <= int(t) < vocab:
                raise StepError(f"token id {t} is outside the vocabulary of {vocab}")
        for w in e.want:
            if not 0 <= int(w) < n:
                raise StepError(f"wanted place {w} is outside the {n} tokens of sequence {b}")
            want_rows.append(cu[-1] + int(w))
        tokens.extend(int(t) for t in e.tokens)
        positions.extend(range(s0, s0 + n))
        token_seq.extend([b] * n)
        cu.append(cu[-1] + n)
        slots.append(e.slot)
        start.append(s0)
    cache.reserve_many([(e.slot, cache.length(e.slot) + len(e.tokens)) for e in entries])
    cache.flush_tables()

    n_tok, n_seq, n_want = len(tokens), len(entries), len(want_rows)
    flat = tokens + positions + token_seq + cu + slots + start + want_rows
    host = torch.tensor(flat, dtype=torch.int32)
    dev = model.rt.device
    if dev.type == "cuda":
        meta = host.pin_memory().to(dev, non_blocking=True)
    else:
        meta = host.to(dev)
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
    )
    rows = take(n_want) if n_want else None
    return ctx, rows


def run_layers(model: Model, cache: Cache, ctx: StepContext) -> ResidualStream:
    """Embedding, then every schedule entry in order."""
    stream = model.embedding.forward(ctx)
    for i, entry in enumerate(model.plan.schedule):
        model.blocks[entry.layer].forward(stream, ctx, cache.handles[i])
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
    ctx, rows = build_context(model, cache, entries)
    stream = run_layers(model, cache, ctx)
    logits = logits_at(model, stream, ctx, rows)
    for e in entries:
        cache.advance(e.slot, len(e.tokens))
    return logits
