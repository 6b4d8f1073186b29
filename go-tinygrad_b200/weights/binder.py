"""Binding tensors to a model by name.

Every part of a model declares the tensors it needs as `WeightSpec`s (full
name as stored in the checkpoint, shape, and what kind of values it holds).
`bind` checks the whole list against a model folder at once and raises one
`WeightError` that lists every missing tensor, every unexpected tensor and
every wrong shape.  The reference binds by the same HF names
(model/llama.go:477-494 and :599-613) but reports only the first missing name
and accepts any shape whose element count matches (model/llama.go:341-349).
"""
from __future__ import annotations

from dataclasses import dataclass
from fnmatch import fnmatchcase
from typing import Dict, Iterable, List, Sequence, Tuple

import torch

from .safetensors_io import TensorSource


@dataclass(frozen=True)
class WeightSpec:
    name: str
    shape: Tuple[int, ...]
    # 'matrix' and 'table' follow the run's compute dtype; 'vector' (norm scales
    # and the like) is always held in float32; 'ignored' may be in the file but
    # is never read.  'std' and 'mean' are what the
    # random-weights mode draws from.
    role: str = "matrix"
    optional: bool = False
    std: float = 0.02
    mean: float = 0.0


class WeightError(ValueError):
    """Tensors of the checkpoint and tensors of the model do not match."""

    def __init__(self, where: str, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 wrong_dtype: Sequence[Tuple[str, str]] = ()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = [f"weights of {where} do not match the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, want, got in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, the model needs {list(want)}")
        for name, got in self.wrong_dtype:
            lines.append(f"  wrong dtype: {name} is {got}, a floating-point tensor is needed")
        super().__init__("\n".join(lines))


def check_specs(specs: Iterable[WeightSpec]) -> List[WeightSpec]:
    out, seen = [], {}
    for s in specs:
        if s.name in seen:
            if seen[s.name].shape != tuple(s.shape):
                raise ValueError(f"two parts declare {s.name!r} with different shapes")
            continue
        seen[s.name] = s
        out.append(s)
    return out


def bind(source: TensorSource, specs: Iterable[WeightSpec], where: str = None,
         ignore: Sequence[str] = (), copy: bool = True) -> Dict[str, torch.Tensor]:
    """Host tensors by name, in their stored dtype, for exactly the declared specs.
    A tensor of the checkpoint that no spec declares is an error unless its name
    matches one of the shell-style patterns in `ignore`.  With copy=False the
    tensors are read-only views of the mapped files, to be used (sent to the
    device) and dropped before `source` is closed."""
    specs = check_specs(specs)
    where = where or source.folder
    missing, wrong_shape, wrong_dtype = [], [], []
    declared = set()
    for s in specs:
        declared.add(s.name)
        if s.name not in source:
            if not s.optional:
                missing.append(s.name)
            continue
        got = tuple(source.shape(s.name))
        if got != tuple(s.shape):
            wrong_shape.append((s.name, tuple(s.shape), got))
        elif not source.dtype(s.name).is_floating_point:
            wrong_dtype.append((s.name, str(source.dtype(s.name))))
    unexpected = sorted(n for n in source.names()
                        if n not in declared and not any(fnmatchcase(n, pat) for pat in ignore))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(where, missing, unexpected, wrong_shape, wrong_dtype)
    return {s.name: source.tensor(s.name, copy=copy) for s in specs
            if s.name in source and s.role != "ignored"}
