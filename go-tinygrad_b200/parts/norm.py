"""RMSNorm, fused with the residual add that precedes it.

y = w * x * (1/sqrt(mean(x^2) + eps)) with the sum of squares and the scale
in float32 (backends/simd/vec.go:72-85).  Parameters: ``size``, ``eps``,
``weight`` (tensor name).
"""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from ..kernels import ops
from ..weights.binder import WeightSpec
from .base import Norm, ResidualStream, Runtime, StepContext, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    def __init__(self, spec):
        super().__init__(spec)
        self.size = int(self.param("size"))
        self.eps = float(self.param("eps"))
        self.weight_name = str(self.param("weight"))
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.weight_name, (self.size,), role="vector", mean=1.0)]

    def load(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        self.weight = rt.vector(tensors[self.weight_name])

    def forward(self, stream: ResidualStream, ctx: StepContext,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n_out = rows.numel() if rows is not None else stream.residual.shape[0]
        out = ctx.rt.empty(n_out, self.size)
        ops.add_rmsnorm(stream.residual, stream.pending, self.weight, self.eps, out, rows)
        if rows is None:
            stream.pending = None
        return out
