"""The generation loop above the step function.

Requests are split into batches that start together (engine/schedule.py).  A
batch's prompts, of unequal lengths, go through one step; then every live
sequence brings one token per step.  A sequence ends at a stop token (which it
keeps), at its token limit or at the model's longest sequence; it leaves the
batch at once and its slot and pages are free for the next batch.  Host tokens
in, host tokens out: each step uploads the tokens it feeds and downloads the
tokens it sampled.

The reference's loop: model/llama.go:1047-1474 (one sequence, exactly
`maxTokens` tokens, greedy).
"""
from __future__ import annotations

import weakref
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple, Union

import torch

from ..cache import Cache
from ..sampling import Sampler
from .decode import DecodeBatch
from .model import Model
from .schedule import SequenceProgress, live, plan_batches
from .step import StepEntry, step


@dataclass
class GenerationResult:
    tokens: List[int]            # the new tokens only
    finish_reason: str           # "stop" | "length" | "capacity"


def _pick(sampler: Sampler, logits: torch.Tensor, seqs: Sequence[SequenceProgress]) -> List[int]:
    dev = logits.device
    ids = torch.tensor([[s.request for s in seqs], [len(s.tokens) for s in seqs]], dtype=torch.int32)
    ids = ids.to(dev, non_blocking=False)
    return sampler.pick(logits, ids[0].contiguous(), ids[1].contiguous()).cpu().tolist()


def generate(model: Model, prompts: Sequence[Sequence[int]],
             max_new_tokens: Union[int, Sequence[int]] = 50, *, temperature: float = 0.0,
             seed: int = 0, stop: Optional[Sequence[int]] = None, cache: Optional[Cache] = None,
             max_batch: Optional[int] = None, max_tokens: Optional[int] = None,
             max_sequence: Optional[int] = None, use_graph: bool = True) -> List[GenerationResult]:
    """Generate for every prompt (lists of token ids).  `stop` defaults to the
    model's own end tokens (config.json's eos_token_id).  With no `cache` one
    is made that holds `max_tokens` tokens (default: what the largest batch
    needs, up to `max_batch` requests at a time, default 64).  `max_sequence`
    caps a sequence's length (prompt and new tokens) below the model's own longest
    position: a request that reaches it ends with "capacity".  Decode steps of a
    batch whose membership does not change are replayed as a CUDA graph (one
    recording per batch size, kept with a `cache` the caller passes, so that
    later calls with the same cache, temperature and seed record nothing) unless
    `use_graph` is False or the model cannot be captured (a part of it talks to
    the host in its forward, or a diagnostic hook is set: `Model.capturable`)."""
    n = len(prompts)
    limits = [int(max_new_tokens)] * n if isinstance(max_new_tokens, int) else [int(m) for m in max_new_tokens]
    if len(limits) != n:
        raise ValueError("max_new_tokens must be one number or one per prompt")
    stop_set = set(model.plan.stop_tokens if stop is None else stop)
    max_seq = model.plan.max_position
    if max_sequence is not None:
        if max_sequence <= 0:
            raise ValueError("max_sequence must be positive")
        max_seq = max_sequence if max_seq is None else min(max_seq, int(max_sequence))
    if cache is not None:
        max_seq = cache.max_sequence if max_seq is None else min(max_seq, cache.max_sequence)
    lengths = [len(p) for p in prompts]
    own_cache = cache is None
    if cache is None:
        max_batch = max_batch or 64
        if max_tokens is None:
            longest = max_seq if max_seq is not None else max(l + m for l, m in zip(lengths, limits))
            need = sorted(((min(l + max(0, m - 1), longest) + 63) // 64 * 64 for l, m in zip(lengths, limits)),
                          reverse=True)
            max_tokens = max(64, sum(need[:max_batch]))
        cache = model.new_cache(max_tokens=max_tokens, max_slots=max_batch)
    max_batch = min(max_batch or cache.n_slots, cache.n_slots)
    batches = plan_batches(lengths, limits, max_tokens=cache.max_tokens, max_batch=max_batch,
                           max_sequence=max_seq)
    sampler = Sampler(temperature, seed)
    results: List[Optional[GenerationResult]] = [None] * n
    # batch size (and what else a recording fixes) -> DecodeBatch
    # A caller who keeps a cache over several calls keeps, with it, the decode batches made
    # for it, so that a later call records nothing anew; they go when the cache goes.
    kept = {} if own_cache else cache.attachments.setdefault("decode_batches", {})
    key = lambda size: (id(model), size, sampler.temperature, sampler.seed, bool(use_graph))

    for batch in batches:
        seqs = [SequenceProgress(i, lengths[i], limits[i], stop_set, max_seq) for i in batch]
        for s in seqs:
            s.start()
        # The longest sequences come first in the batch, in the prompt step and in every
        # decode step: kernels hand out their blocks sequence by sequence in batch
        # order, and the long ones should not be the last to start.  Sequences grow
        # together, so the order holds while the batch lives.
        running = sorted(live(seqs), key=lambda s: -s.prompt_length)
        slots = {s.request: cache.open_sequence() for s in running}
        try:
            if running:
                entries = [StepEntry(slots[s.request], prompts[s.request], [lengths[s.request] - 1])
                           for s in running]
                logits = step(model, cache, entries)
                for s, tok in zip(running, _pick(sampler, logits, running)):
                    s.accept(tok)
            decode, members = None, None
            while True:
                for s in running:
                    if s.finished and s.request in slots:
                        cache.close_sequence(slots.pop(s.request))
                running = live(running)
                if not running:
                    break
                now = tuple(s.request for s in running)
                if now != members:          # the batch shrank: another fixed set of sequences
                    decode = kept.get(key(len(now)))
                    if decode is None or decode.model is not model:
                        # one recorded step per batch size serves every set of that size
                        # (a batch that is kept with the caller's cache refers to it weakly: the two
                        # go together when the caller lets go of the cache, without the collector's help)
                        decode = kept[key(len(now))] = DecodeBatch(model, cache if own_cache else weakref.proxy(cache),
                                                                   [slots[r] for r in now], now, sampler,
                                                                   use_graph=use_graph)
                    else:
                        decode.rebind([slots[r] for r in now], now)
                    members = now
                picked = decode.step_host([s.tokens[-1] for s in running], [len(s.tokens) for s in running])
                for s, tok in zip(running, picked):
                    s.accept(tok)
        finally:
            for slot in slots.values():
                cache.close_sequence(slot)
        for s in seqs:
            results[s.request] = GenerationResult(s.tokens, s.finish_reason or "length")
    return results  # type: ignore[return-value]
