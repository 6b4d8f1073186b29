"""Position encodings.

``rotary``: rotation of half-split pairs (i, i + head_dim/2) of queries and keys
by the angle position * f_i, f_i = theta^(-2i/head_dim) (model/llama.go:838-865
for the table, :1556-1589 for the pairing).  The frequencies are computed once
in float64 on the host; the angles of a step's tokens are computed on the
device as float64 products and rounded to float32 (cos, sin) pairs, once per
step, and shared by all layers that use equal parameters.  Parameters:
``head_dim``, ``theta``, ``scaling`` (None or the llama3 block: factor,
low_freq_factor, high_freq_factor, original_max_position_embeddings), and
optionally ``pairing`` ("half", the default: channel i with i + d/2;
"interleaved": 2i with 2i+1) and ``rotary_dim`` (d: how many of a head's first
channels rotate; default all; f_i = theta^(-2i/d)).  The rotation inside the
prompt projection and inside the decode attention serves the default layout;
any other is rotated by the general kernel between projection and attention.

The llama3 scaling is not in the reference: wavelengths shorter than
original/high_freq_factor keep their frequency, longer than
original/low_freq_factor are divided by `factor`, and those in between are
blended linearly.

``none``: no position encoding.
"""
from __future__ import annotations

import math
from typing import Mapping, Optional

import torch

from ..kernels import ops
from .base import PositionEncoding, Runtime, StepContext, register_part


def rotary_frequencies(head_dim: int, theta: float, scaling: Optional[Mapping] = None):
    """float64 list of head_dim/2 frequencies."""
    freqs = [1.0 / math.pow(theta, (2 * i) / head_dim) for i in range(head_dim // 2)]
    if scaling:
        factor = float(scaling["factor"])
        low = float(scaling["low_freq_factor"])
        high = float(scaling["high_freq_factor"])
        original = float(scaling["original_max_position_embeddings"])
        scaled = []
        for f in freqs:
            wavelength = 2.0 * math.pi / f
            if wavelength < original / high:
                scaled.append(f)
            elif wavelength > original / low:
                scaled.append(f / factor)
            else:
                smooth = (original / wavelength - low) / (high - low)
                scaled.append((1.0 - smooth) * f / factor + smooth * f)
        freqs = scaled
    return freqs


@register_part("position", "rotary")
class RotaryEncoding(PositionEncoding):
    def __init__(self, spec):
        super().__init__(spec)
        self.head_dim = int(self.param("head_dim"))
        self.theta = float(self.param("theta"))
        scaling = self.p.get("scaling")
        self.scaling = dict(scaling) if scaling else None
        self.pairing = str(self.p.get("pairing") or "half")
        if self.pairing not in ("half", "interleaved"):
            raise ValueError(f"rotary pairing {self.pairing!r} is not known: 'half' or 'interleaved'")
        self.rotary_dim = int(self.p.get("rotary_dim") or self.head_dim)
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary encoding needs an even number of rotated channels up to the head's "
                             f"{self.head_dim}, got {self.rotary_dim}")
        self._key = ("rotary", self.rotary_dim, self.theta,
                     tuple(sorted(self.scaling.items())) if self.scaling else None)
        self.inv_freq: Optional[torch.Tensor] = None

    def load(self, tensors, rt: Runtime) -> None:
        self.inv_freq = torch.tensor(rotary_frequencies(self.rotary_dim, self.theta, self.scaling),
                                     dtype=torch.float64, device=rt.device)

    def rotation(self, ctx: StepContext) -> Optional[torch.Tensor]:
        table = ctx.shared.get(self._key)
        if table is None:
            table = ctx.rt.empty(ctx.n_tokens, self.rotary_dim // 2, 2, dtype=torch.float32, lifetime="step")
            ops.rope_table(ctx.positions, self.inv_freq, table)
            ctx.shared[self._key] = table
        return table


@register_part("position", "none")
class NoPosition(PositionEncoding):
    pass
