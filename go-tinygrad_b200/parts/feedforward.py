"""Dense gated feed-forward (SwiGLU): down(silu(gate(x)) * up(x)), silu(g) =
g / (1 + exp(-g)) (model/llama.go:1361-1401, backends/simd/vec.go:52-59).

Parameters: ``hidden_size``, ``intermediate_size`` and the tensor names
``gate``, ``up``, ``down``.  Gate and up are fused at load into one matrix
[2 * intermediate, hidden] so that one product serves both: in float32 the gate
rows come first and a second kernel applies the activation; in bfloat16 the rows
alternate in blocks of 8 gate and 8 up features and the product's epilogue
applies the activation to its float accumulators.
"""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from ..kernels import ops
from ..weights.binder import WeightSpec
from .base import FeedForward, Runtime, StepContext, emit_update, register_part


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.param("hidden_size"))
        self.inter = int(self.param("intermediate_size"))
        self.names = {k: str(self.param(k)) for k in ("gate", "up", "down")}
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.names["gate"], (self.inter, self.hidden)),
                WeightSpec(self.names["up"], (self.inter, self.hidden)),
                WeightSpec(self.names["down"], (self.hidden, self.inter))]

    def load(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        gate, up = tensors[self.names["gate"]].to(rt.dtype), tensors[self.names["up"]].to(rt.dtype)
        # bfloat16: gate and up rows interleaved in blocks of 8 so that the product's
        # epilogue can apply silu(gate) * up to its float accumulators and write the
        # activation directly; float32: gate rows then up rows, and a kernel of its own
        self.fused = rt.dtype == torch.bfloat16 and self.inter % 8 == 0
        if self.fused:
            self.w_gate_up = rt.matrix(ops.interleave_gate_up(gate, up))
        else:
            self.w_gate_up = rt.matrix(torch.cat([gate, up], dim=0))
        self.w_down = rt.matrix(tensors[self.names["down"]])

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        rt = ctx.rt
        n = x.shape[0]
        act = rt.empty(n, self.inter)
        if self.fused:
            ops.linear(x, self.w_gate_up, act, epilogue="swiglu")
        else:
            gate_up = rt.empty(n, 2 * self.inter)
            ops.linear(x, self.w_gate_up, gate_up)
            ctx.trace("gate_pre", gate_up[:, : self.inter])
            ctx.trace("up", gate_up[:, self.inter:])
            ops.swiglu(gate_up, act)
        ctx.trace("gate_act", act)
        return emit_update(act, self.w_down, ctx)
