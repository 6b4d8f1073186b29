"""Choosing the next token from float32 logits, on the device.

``temperature == 0``: greedy, the first index of the maximum
(model/inference_helpers.go:153-166) -- the only rule the reference has.
``temperature > 0``: softmax(logits / temperature) and an inverse-CDF draw with
a uniform that is a function of (seed, request index, step) alone, so that a
request draws the same tokens alone or in any batch.
"""
from __future__ import annotations

import torch

from ..kernels import ops

_M64 = (1 << 64) - 1


def _mix64(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def uniform(seed: int, request: int, step: int) -> float:
    """The uniform in [0, 1) the sampling kernel uses for (seed, request, step)."""
    z = _mix64(seed & _M64)
    z = _mix64(z ^ ((request * 0xD1B54A32D192ED03) & _M64))
    z = _mix64(z ^ ((step * 0x8CB92BA72F3D8DD7) & _M64))
    return (z >> 40) * (1.0 / (1 << 24))


class Sampler:
    def __init__(self, temperature: float = 0.0, seed: int = 0):
        if temperature < 0:
            raise ValueError("the temperature must not be negative")
        self.temperature = float(temperature)
        self.seed = int(seed)

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0

    def pick(self, logits: torch.Tensor, requests: torch.Tensor, steps: torch.Tensor,
             out: torch.Tensor = None) -> torch.Tensor:
        """int32 [rows]: one token per row of `logits`; `requests` and `steps`
        (int32, on the device) say whose draw each row is."""
        if out is None:
            out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
        if self.greedy:
            ops.argmax(logits, out)
        else:
            ops.sample_temperature(logits, self.temperature, self.seed, requests, steps, out)
        return out


__all__ = ["Sampler", "uniform"]
