"""The generation loop's decisions, as plain host code without a device:
which requests form the next batch, and when a sequence ends.

The reference generates one sequence at a time for exactly `maxTokens` tokens
and has no stop tokens in its loop (model/llama.go:1047-1053,1474; its
front-ends cut the text at an end marker afterwards,
cmd/llmchat/main.go:135-151).  Batches, stop tokens and sequences that end
earlier are this library's.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Iterable, List, Optional, Sequence, Set

PAGE_TOKENS = 64


def _rounded(n: int) -> int:
    return (n + PAGE_TOKENS - 1) // PAGE_TOKENS * PAGE_TOKENS


class RequestTooLarge(ValueError):
    """One request alone does not fit the cache."""


def plan_batches(prompt_lengths: Sequence[int], max_new_tokens: Sequence[int], *, max_tokens: int,
                 max_batch: int, max_sequence: Optional[int] = None) -> List[List[int]]:
    """Split requests, in order, into batches that start together.  A batch holds
    at most `max_batch` requests and its requests' worst-case footprints
    (prompt + new tokens, each rounded up to a page) fit `max_tokens`.  A
    request whose worst case exceeds `max_sequence` positions is still taken:
    it ends when it reaches that length."""
    if max_batch <= 0:
        raise ValueError("max_batch must be positive")
    batches: List[List[int]] = []
    current: List[int] = []
    used = 0
    for i, (p, n) in enumerate(zip(prompt_lengths, max_new_tokens)):
        if p <= 0:
            raise ValueError(f"request {i} has an empty prompt")
        if n < 0:
            raise ValueError(f"request {i} asks for a negative number of tokens")
        total = p + max(0, n - 1)          # the last generated token is never fed back
        if max_sequence is not None:
            if p > max_sequence:
                raise RequestTooLarge(f"request {i}: a prompt of {p} tokens exceeds the longest "
                                      f"sequence the model takes ({max_sequence})")
            total = min(total, max_sequence)
        need = _rounded(total)
        if need > max_tokens:
            raise RequestTooLarge(f"request {i} needs room for {need} tokens; the cache holds {max_tokens}")
        if current and (len(current) >= max_batch or used + need > max_tokens):
            batches.append(current)
            current, used = [], 0
        current.append(i)
        used += need
    if current:
        batches.append(current)
    return batches


@dataclass
class SequenceProgress:
    """What the loop knows about one request while its batch runs."""
    request: int                  # index among all requests (keys the sampler's draws)
    prompt_length: int
    max_new_tokens: int
    stop: Set[int]
    max_sequence: Optional[int] = None
    tokens: List[int] = field(default_factory=list)
    finish_reason: Optional[str] = None

    @property
    def finished(self) -> bool:
        return self.finish_reason is not None

    def start(self) -> None:
        if self.max_new_tokens == 0:
            self.finish_reason = "length"

    def accept(self, token: int) -> None:
        """Take the token sampled for this sequence and decide whether it goes on."""
        if self.finished:
            raise RuntimeError("a finished sequence was given another token")
        self.tokens.append(int(token))
        if int(token) in self.stop:
            self.finish_reason = "stop"
        elif len(self.tokens) >= self.max_new_tokens:
            self.finish_reason = "length"
        elif (self.max_sequence is not None
              and self.prompt_length + len(self.tokens) > self.max_sequence):
            # feeding this token back would need a position the model does not have
            self.finish_reason = "capacity"


def live(progress: Iterable[SequenceProgress]) -> List[SequenceProgress]:
    return [p for p in progress if not p.finished]
