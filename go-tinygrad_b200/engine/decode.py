"""A fixed set of sequences decoding together: one token each per step, with
the step captured once as a CUDA graph and replayed.

The decode step of a batch is launch-bound (a few hundred small kernels), so it
is recorded once -- embedding, every layer from the cache, final norm, head and
the choice of the next token -- and replayed from buffers at fixed addresses:
tokens, positions, the count of tokens each sequence has generated (it keys the
random draw) and the sampled tokens.  Two ways to drive it:

  * `step_host(tokens)`: the host uploads the tokens to feed, runs the step and
    downloads the sampled tokens (what the generation loop does);
  * `step_device()`: the sampled tokens become the next input on the device and
    nothing crosses the bus (a kernel moves them; for timing the step itself).

The first run of a batch executes eagerly (it loads and configures kernels,
which a capture must not do), the second is captured.  A recording fixes what
the parts chose from the batch's longest sequence (into how many blocks the
keys of a sequence are split; a sequence that outgrows the plan is still computed
right, in larger parts): it is made again when the sequences have outgrown it by
a sixth, or when the
object is given much shorter sequences (`rebind`).  Which sequences the batch
holds is data (slots and request ids in a device buffer), so one recording
serves every set of as many sequences.
"""
from __future__ import annotations

import gc
from typing import List, Optional, Sequence

import torch

from ..cache import Cache
from ..kernels import ops
from ..parts.base import StepContext
from ..sampling import Sampler
from .model import Model
from .step import logits_at, run_layers


class DecodeBatch:
    def __init__(self, model: Model, cache: Cache, slots: Sequence[int], requests: Sequence[int],
                 sampler: Sampler, use_graph: bool = True, chained: bool = True):
        self.model, self.cache, self.sampler = model, cache, sampler
        self.slots = list(slots)
        B = self.B = len(self.slots)
        dev = model.rt.device
        # one device buffer, views at fixed addresses
        #   tokens | positions | steps | token_seq | cu_seqlens | slots | requests | rows
        self.meta = torch.zeros(8 * B + 1, dtype=torch.int32, device=dev)
        cut = lambda a, n: self.meta[a:a + n]
        self.tokens, self.positions, self.steps = cut(0, B), cut(B, B), cut(2 * B, B)
        self.token_seq, self.cu = cut(3 * B, B), cut(4 * B, B + 1)
        self.slot_ids, self.requests, self.rows = cut(5 * B + 1, B), cut(6 * B + 1, B), cut(7 * B + 1, B)
        ar = torch.arange(B + 1, dtype=torch.int32)
        fixed = torch.cat([ar[:B], ar, torch.tensor(self.slots, dtype=torch.int32),
                           torch.tensor(list(requests), dtype=torch.int32), ar[:B]])
        self.meta[3 * B:].copy_(fixed.to(dev))
        self.sampled = torch.zeros(B, dtype=torch.int32, device=dev)
        pin = dev.type == "cuda"
        self.h_in = torch.zeros(3 * B, dtype=torch.int32, pin_memory=pin)
        self.h_out = torch.zeros(B, dtype=torch.int32, pin_memory=pin)
        self._h_in, self._h_out = self.h_in.numpy(), self.h_out.numpy()   # the same memory, cheap to fill and read
        self.logits: Optional[torch.Tensor] = None
        # a part that talks to the host in its forward, or a listening diagnostic hook,
        # cannot be recorded: such a model's steps are launched kernel by kernel
        self.use_graph = use_graph and dev.type == "cuda" and model.capturable
        self.chained = chained and dev.type == "cuda"     # kernels of the step overlap their launch gaps
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self._runs = 0
        self._planned_len = 0                             # the longest sequence the recording was made for
        self._planned_total = 0                           # ... and all sequences' lengths together
        self._open_first = False                          # the next step runs in the open before one is recorded again

    def rebind(self, slots: Sequence[int], requests: Sequence[int]) -> None:
        """The same number of sequences, other slots and request ids: the
        recorded step is kept."""
        if len(slots) != self.B or len(requests) != self.B:
            raise ValueError(f"this decode batch holds {self.B} sequences")
        self.slots = list(slots)
        B = self.B
        fixed = torch.tensor(list(slots) + list(requests), dtype=torch.int32)
        self.meta[5 * B + 1:7 * B + 1].copy_(fixed.to(self.meta.device))

    # ------------------------------------------------------------------ state
    def set_state(self, tokens: Sequence[int], steps: Sequence[int]) -> None:
        """Tokens to feed next and how many tokens each sequence has generated;
        positions are the sequences' lengths in the cache."""
        B, h, length = self.B, self._h_in, self.cache.length
        h[:B] = tokens
        h[B:2 * B] = [length(s) for s in self.slots]
        h[2 * B:] = steps
        self.meta[:3 * B].copy_(self.h_in, non_blocking=True)

    def _context(self) -> StepContext:
        return StepContext(rt=self.model.rt, n_tokens=self.B, n_seqs=self.B, tokens=self.tokens,
                           positions=self.positions, token_seq=self.token_seq, cu_seqlens=self.cu,
                           slots=self.slot_ids, start_pos=self.positions, max_q_len=1,
                           max_kv_len=self._planned_len, is_decode=True, total_kv_len=self._planned_total,
                           step=self.model.steps_run, op_hook=self.model.op_hook)

    def _forward(self) -> None:
        self.model.rt.workspace.begin_step()
        ctx = self._context()
        with ops.chained_launches(self.chained), ops.checked_access(self.model.rt.check_access):
            stream = run_layers(self.model, self.cache, ctx)
            self.logits = logits_at(self.model, stream, ctx, self.rows)
            self.sampler.pick(self.logits, self.requests, self.steps, out=self.sampled)

    def _launch(self) -> None:
        """Run the step for the state now on the device; grows every sequence by one."""
        self.cache.reserve_many([(s, self.cache.length(s) + 1) for s in self.slots])
        self.cache.flush_tables()
        lengths = [self.cache.length(s) + 1 for s in self.slots]
        longest = max(lengths)
        if self.model.op_hook is not None or self.model.rt.check_access:   # a hook listens or checks run: in the open
            self.graph = None
            self._planned_len, self._planned_total = longest, sum(lengths)
            self._forward()
            self._finish_step()
            return
        if self.graph is None or not self.use_graph:
            self._planned_len, self._planned_total = longest, sum(lengths)
        elif longest > self._planned_len * 1.17 or longest * 2 < self._planned_len:
            self.graph = None                             # outgrown (or far too long a plan): record again,
            self._open_first = True                       # after one step in the open with the new plan
            self._planned_len, self._planned_total = longest, sum(lengths)
        if not self.use_graph:
            self._forward()
        elif self.graph is not None:
            self.graph.replay()
        elif self._runs == 0 or self._open_first:
            self._open_first = False
            self._forward()
        else:
            self.graph = self._record()
            self.graph.replay()
        self._finish_step()

    def _finish_step(self) -> None:
        self._runs += 1
        self.model.steps_run += 1
        for s in self.slots:
            self.cache.advance(s, 1)

    def _record(self) -> "torch.cuda.CUDAGraph":
        """Capture one step on a side stream.  Done by hand rather than with
        `torch.cuda.graph`, which first collects garbage and hands every cached block
        back to the driver: a generation loop records a step whenever its batch
        shrinks, and would pay for both each time (and allocate its cache anew)."""
        graph = torch.cuda.CUDAGraph()
        main = torch.cuda.current_stream()
        if DecodeBatch._side is None:
            DecodeBatch._side = torch.cuda.Stream()
        side = DecodeBatch._side
        side.wait_stream(main)
        # the recording addresses the workspace's buffers: they stay alive with this object
        # even if a later, larger step makes the workspace replace them
        self.model.rt.workspace.begin_step()              # grown now, to what the run before asked for
        self._workspace_held = self.model.rt.workspace.buffers()
        # While a recording runs, nothing else may talk to the device: a graph or a tensor
        # that the cyclic collector happens to finalise in the middle of it (garbage of
        # earlier work, of this library's or of the caller's) frees device memory and
        # invalidates the recording.  So the collector rests meanwhile (it is not run first,
        # as torch.cuda.graph does: that costs more than the recording).
        collecting = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.stream(side):
                graph.capture_begin()
                try:
                    self._forward()
                finally:
                    graph.capture_end()
        finally:
            if collecting:
                gc.enable()
            main.wait_stream(side)
        return graph

    _side: Optional["torch.cuda.Stream"] = None

    # ------------------------------------------------------------------ driving
    def step_host(self, tokens: Sequence[int], steps: Sequence[int]) -> List[int]:
        self.set_state(tokens, steps)
        self._launch()
        self.h_out.copy_(self.sampled, non_blocking=True)
        if self.model.rt.device.type == "cuda":
            torch.cuda.current_stream().synchronize()
        return self._h_out.tolist()

    def step_device(self) -> None:
        """Feed back the tokens just sampled; no host synchronisation."""
        ops.advance(self.tokens, self.positions, self.steps, self.sampled)
        self._launch()

    def reserve_ahead(self, n_steps: int) -> None:
        """Take the pages `n_steps` more steps will need now, so that the steps
        themselves touch no block table."""
        self.cache.reserve_many([(s, self.cache.length(s) + n_steps) for s in self.slots])
        self.cache.flush_tables()
