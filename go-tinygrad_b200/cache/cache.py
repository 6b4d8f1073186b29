"""The cache of a model: keys and values per layer run, per-sequence state of
fixed size, and the slots that tie both to sequences.

What a mixer needs is a *request*: `KVRequest` (keys and values of so many
heads of such a size, all of them or a window) or `StateRequest` (a record of
fixed shape per sequence).  Runs whose KV requests are equal form a *group*
with storage of its own -- its own pages, page pool and block table -- so that
layers that keep every key and layers that keep a window do not share storage.

Storage of a group: ``pages[entry, page, 0|1, kv_head, token(64), channel]``
(keys at 0, values at 1).  ``block_table[slot, i]`` is the page holding tokens
``[64*i, 64*i+64)`` of the sequence in `slot`.  A sequence holds
ceil(length/64) pages per group -- a group that keeps a window gives back, as
the sequence grows, the pages that have slid out of it -- and pages and the
slot return to the free lists when the sequence is closed, and are handed out
again.

The reference keeps one growing slice (CPU) or one 2048-position buffer (GPU)
per layer for its single sequence (model/llama.go:984-985,1017-1029;
model/gpu_forward.go:477-496); per-layer widths for layers that reuse another
layer's cache are in model/kv_staging.go:11-54.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple, Union

import torch

from .pages import CacheFull, CacheMisuse, PagePool, SlotTable

PAGE_TOKENS = 64


@dataclass(frozen=True)
class KVRequest:
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None      # None: every key is kept


@dataclass(frozen=True)
class StateRequest:
    name: str
    shape: Tuple[int, ...]
    dtype: str = "float32"            # "float32" | "bfloat16" | "int32"


Request = Union[KVRequest, StateRequest]
_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


class KVEntryView:
    """What a kernel needs to address one run's keys and values."""
    __slots__ = ("k", "v", "page_stride", "block_table", "table_stride", "n_kv_heads", "head_dim",
                 "window")

    def __init__(self, k, v, block_table, n_kv_heads, head_dim, window):
        self.k, self.v = k, v
        self.page_stride = k.stride(0)
        self.block_table = block_table
        self.table_stride = block_table.stride(0)
        self.n_kv_heads, self.head_dim, self.window = n_kv_heads, head_dim, window


class CacheHandle:
    """The storage of one schedule entry: `.kv` (or None) and `.state(name)`.
    `writes` is False when the entry reads another entry's storage."""

    def __init__(self, kv: Optional[KVEntryView], states: Dict[str, torch.Tensor], writes: bool):
        self.kv = kv
        self._states = states
        self.writes = writes

    def state(self, name: str) -> torch.Tensor:
        """[n_slots, *shape]; row `slot` belongs to the sequence in that slot."""
        return self._states[name]


class _KVGroup:
    def __init__(self, request: KVRequest, n_entries: int, n_pages: int, n_slots: int,
                 pages_per_seq: int, dtype: torch.dtype, device: torch.device):
        self.request = request
        self.pool = PagePool(n_pages)
        self.storage = torch.zeros((n_entries, n_pages, 2, request.n_kv_heads, PAGE_TOKENS,
                                    request.head_dim), dtype=dtype, device=device)
        self.table_host = torch.zeros((n_slots, pages_per_seq), dtype=torch.int32)
        if device.type == "cuda":
            self.table_host = self.table_host.pin_memory()
        self.table = torch.zeros((n_slots, pages_per_seq), dtype=torch.int32, device=device)
        self.pages_of: Dict[int, List[int]] = {}     # slot -> its pages by index; -1: given back (slid out of the window)
        self.dirty: set = set()

    def view(self, entry: int) -> KVEntryView:
        s = self.storage[entry]
        return KVEntryView(s[:, 0], s[:, 1], self.table, self.request.n_kv_heads,
                           self.request.head_dim, self.request.window)


class Cache:
    """`requests[i]` lists what schedule entry i needs (empty for an entry that
    reads another entry's storage: then `shared_from[i]` names that entry)."""

    def __init__(self, requests: Sequence[Sequence[Request]], shared_from: Sequence[Optional[int]],
                 *, max_tokens: int, max_slots: Optional[int] = None, max_position: Optional[int] = None,
                 dtype: torch.dtype, device: Union[str, torch.device]):
        self.device = torch.device(device)
        self.dtype = dtype
        if max_tokens <= 0:
            raise ValueError("max_tokens must be positive")
        self.n_pages = (max_tokens + PAGE_TOKENS - 1) // PAGE_TOKENS
        self.max_tokens = self.n_pages * PAGE_TOKENS
        self.n_slots = max_slots if max_slots is not None else min(self.n_pages, 1024)
        per_seq = self.n_pages
        if max_position is not None:
            per_seq = min(per_seq, (max_position + PAGE_TOKENS - 1) // PAGE_TOKENS)
        self.pages_per_seq = max(1, per_seq)
        # the longest sequence, in tokens: what the pages of one sequence hold, and no
        # more than the model's own longest position where one is given
        self.max_sequence = self.pages_per_seq * PAGE_TOKENS
        if max_position is not None:
            self.max_sequence = min(self.max_sequence, int(max_position))
        self.slots = SlotTable(self.n_slots)
        self._length = [0] * self.n_slots
        # what users of the cache keep with it and want gone when it goes (the generation
        # loop: its recorded decode steps); the cache itself never looks inside
        self.attachments: Dict[str, object] = {}

        # group the KV requests
        keys: List[KVRequest] = []
        members: Dict[KVRequest, List[int]] = {}
        for i, reqs in enumerate(requests):
            for r in reqs:
                if isinstance(r, KVRequest):
                    if r not in members:
                        members[r] = []
                        keys.append(r)
                    members[r].append(i)
        self.groups: List[_KVGroup] = []
        kv_of_entry: Dict[int, Tuple[int, int]] = {}
        for r in keys:
            grp = _KVGroup(r, len(members[r]), self.n_pages, self.n_slots, self.pages_per_seq,
                           dtype, self.device)
            for j, i in enumerate(members[r]):
                if i in kv_of_entry:
                    raise ValueError(f"schedule entry {i} asks for two key/value stores")
                kv_of_entry[i] = (len(self.groups), j)
            self.groups.append(grp)

        # fixed-size state
        self._state_tensors: List[torch.Tensor] = []
        states_of_entry: Dict[int, Dict[str, torch.Tensor]] = {}
        for i, reqs in enumerate(requests):
            for r in reqs:
                if isinstance(r, StateRequest):
                    if r.dtype not in _STATE_DTYPES:
                        raise ValueError(f"state dtype {r.dtype!r} is not supported")
                    t = torch.zeros((self.n_slots,) + tuple(r.shape), dtype=_STATE_DTYPES[r.dtype],
                                    device=self.device)
                    states_of_entry.setdefault(i, {})[r.name] = t
                    self._state_tensors.append(t)

        self.handles: List[CacheHandle] = []
        for i in range(len(requests)):
            src = shared_from[i]
            owner = i if src is None else src
            kv = None
            if owner in kv_of_entry:
                g, j = kv_of_entry[owner]
                kv = self.groups[g].view(j)
            self.handles.append(CacheHandle(kv, states_of_entry.get(owner, {}), writes=src is None))

    # ------------------------------------------------------------ sequences
    def open_sequence(self) -> int:
        """A free slot with length 0 and zeroed fixed-size state."""
        slot = self.slots.alloc()
        self._length[slot] = 0
        for grp in self.groups:
            grp.pages_of[slot] = []
        for t in self._state_tensors:
            t[slot].zero_()
        return slot

    def close_sequence(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise CacheMisuse(f"slot {slot} is closed but is not open")
        for grp in self.groups:
            grp.pool.free([p for p in grp.pages_of.pop(slot) if p >= 0], slot)
        self._length[slot] = 0
        self.slots.free(slot)

    def length(self, slot: int) -> int:
        return self._length[slot]

    def reserve(self, slot: int, new_length: int) -> None:
        """Make room for the sequence in `slot` to grow to `new_length` tokens."""
        if not self.slots.is_held(slot):
            raise CacheMisuse(f"slot {slot} is not open")
        need = (new_length + PAGE_TOKENS - 1) // PAGE_TOKENS
        if new_length > self.max_sequence:
            raise CacheFull(f"a sequence of {new_length} tokens exceeds the longest the cache "
                            f"holds ({self.max_sequence})")
        for grp in self.groups:
            have = grp.pages_of[slot]
            if need > len(have):
                if need - len(have) > grp.pool.n_free:
                    raise CacheFull(f"the cache is full: growing a sequence to {new_length} tokens "
                                    f"needs {need - len(have)} more pages of 64 tokens, "
                                    f"{grp.pool.n_free} of {grp.pool.n_pages} are free")
        for grp in self.groups:
            have = grp.pages_of[slot]
            if need > len(have):
                new = grp.pool.alloc(need - len(have), slot)
                grp.table_host[slot, len(have):need] = torch.tensor(new, dtype=torch.int32)
                have.extend(new)
                grp.dirty.add(slot)

    def reserve_many(self, wanted: Sequence[Tuple[int, int]]) -> None:
        """`reserve` for several (slot, new_length) pairs: all of them or none."""
        for grp in self.groups:
            need = 0
            for slot, new_length in wanted:
                if not self.slots.is_held(slot):
                    raise CacheMisuse(f"slot {slot} is not open")
                pages = (new_length + PAGE_TOKENS - 1) // PAGE_TOKENS
                if new_length > self.max_sequence:
                    raise CacheFull(f"a sequence of {new_length} tokens exceeds the longest the "
                                    f"cache holds ({self.max_sequence})")
                need += max(0, pages - len(grp.pages_of[slot]))
            if need > grp.pool.n_free:
                raise CacheFull(f"the cache is full: this step needs {need} more pages of 64 tokens, "
                                f"{grp.pool.n_free} of {grp.pool.n_pages} are free")
        for slot, new_length in wanted:
            self.reserve(slot, new_length)

    def advance(self, slot: int, n_tokens: int) -> None:
        """Record that `n_tokens` more tokens of the sequence are in the cache."""
        new_length = self._length[slot] + n_tokens
        for grp in self.groups:
            if new_length > len(grp.pages_of[slot]) * PAGE_TOKENS:
                raise CacheMisuse(f"slot {slot} advanced to {new_length} tokens without reserved pages")
        self._length[slot] = new_length
        # A group that keeps a window gives back the pages no later token can see: the next
        # token, at position new_length, reaches back to new_length - window + 1.  Their
        # table entries stay as they are; no kernel reads a page before a window's first.
        for grp in self.groups:
            window = grp.request.window
            if window is None:
                continue
            have = grp.pages_of[slot]
            gone = [i for i in range(min(len(have), max(0, new_length - window + 1) // PAGE_TOKENS)) if have[i] >= 0]
            if gone:
                grp.pool.free([have[i] for i in gone], slot)
                for i in gone:
                    have[i] = -1

    def truncate(self, slot: int, new_length: int) -> None:
        """Forget the tokens after `new_length` (their pages stay with the sequence).
        Keys and values are addressed by position, so a shorter length is all it
        takes (the reference's rollback does the same: runtime/kv/staging.go:35-68).
        A record of fixed size has already absorbed the tokens to be forgotten and
        cannot give them back: a cache that holds such state refuses, since a shorter
        length beside an unchanged record would be silently wrong."""
        if self._state_tensors and new_length != self._length[slot]:
            raise CacheMisuse("this cache holds per-sequence state of fixed size, which cannot be "
                              "rolled back by shortening a length; close the sequence and run it again")
        if not 0 <= new_length <= self._length[slot]:
            raise CacheMisuse(f"cannot truncate slot {slot} from {self._length[slot]} to {new_length}")
        for grp in self.groups:
            window = grp.request.window
            if window is not None and any(p < 0 for p in grp.pages_of[slot][max(0, new_length - window + 1) // PAGE_TOKENS:
                                                                         (new_length + PAGE_TOKENS - 1) // PAGE_TOKENS]):
                raise CacheMisuse(f"slot {slot} cannot go back to {new_length} tokens: a layer that keeps a window "
                                  f"of {window} keys has given back pages that length would need")
        self._length[slot] = new_length

    def flush_tables(self) -> None:
        """Copy block-table rows that changed on the host to the device."""
        for grp in self.groups:
            for slot in sorted(grp.dirty):
                grp.table[slot].copy_(grp.table_host[slot])
            grp.dirty.clear()

    # ------------------------------------------------------------ accounting
    def tokens_held(self) -> int:
        """Tokens of capacity that live sequences hold (each rounded up to 64)."""
        if not self.groups:
            return 0
        return max(sum(sum(1 for p in pages if p >= 0) for pages in grp.pages_of.values())
                   for grp in self.groups) * PAGE_TOKENS

    def free_pages(self) -> List[int]:
        return [grp.pool.n_free for grp in self.groups]

    def open_slots(self) -> List[int]:
        return self.slots.held()

    def bytes(self) -> int:
        total = sum(g.storage.numel() * g.storage.element_size() for g in self.groups)
        return total + sum(t.numel() * t.element_size() for t in self._state_tensors)
