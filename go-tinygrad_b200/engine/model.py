"""A model: the parts a plan names, with their weights on the device.

`Model.load(folder)` reads config.json, finds the architecture in the registry,
builds the plan and the parts, binds the checkpoint's tensors by name and hands
each part its own.  The model owns no sequence state: that lives in a `Cache`
(`new_cache`), and `step` (engine/step.py) runs tokens through both.

The reference's loader for comparison: model/llama.go:190-836.
"""
from __future__ import annotations

from typing import Any, List, Mapping, Optional, Sequence, Union

import torch

from ..cache import Cache
from ..config.registry import Architecture, find_architecture, read_config_json
from ..parts.base import Block, Runtime, build_part, walk
from ..parts.plan import ModelPlan, plan_weight_specs
from ..weights.binder import WeightSpec, bind, check_specs
from ..weights.random_init import random_tensors
from ..weights.safetensors_io import TensorSource

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}


def compute_dtype(dtype: Union[str, torch.dtype]) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype in (torch.bfloat16, torch.float32):
            return dtype
    elif dtype in _DTYPES:
        return _DTYPES[dtype]
    raise ValueError(f"dtype must be 'bfloat16' or 'float32', got {dtype!r}")


class Model:
    def __init__(self, plan: ModelPlan, rt: Runtime, config: Any = None):
        plan.check()
        self.plan = plan
        self.rt = rt
        self.config = config
        self.embedding = build_part("embedding", plan.embedding)
        # a block builds and owns what its layer is made of (norms, mixer, feed-forward, ...)
        self.blocks: List[Block] = [build_part("block", layer.block) for layer in plan.layers]
        self.final_norm = build_part("norm", plan.final_norm)
        self.head = build_part("head", plan.head)
        self.loaded = False
        self.steps_run = 0
        # Optional diagnostic: op_hook(step, layer, op, tensor) receives named
        # intermediate values of every layer (see StepContext.trace), as the reference's
        # debugOpHook does (model/debug_hooks.go:5-7).  None in normal execution; while
        # it is set, decode steps are not recorded as CUDA graphs.
        self.op_hook = None

    # ------------------------------------------------------------------ parts
    def parts(self):
        """Every part of the model: each root, then what it owns."""
        for root in (self.embedding, *self.blocks, self.final_norm, self.head):
            yield from walk(root)

    @property
    def capturable(self) -> bool:
        """Whether a step of this model can be recorded as a CUDA graph: every part
        says so, no diagnostic hook listens and no access checks run."""
        return (self.op_hook is None and not self.rt.check_access
                and all(part.capturable for part in self.parts()))

    def weight_specs(self) -> List[WeightSpec]:
        specs: List[WeightSpec] = []
        for part in self.parts():
            specs += part.weight_specs()
        return check_specs(specs)

    def load_tensors(self, tensors: Mapping[str, torch.Tensor]) -> "Model":
        """Give every part the tensors it declared (host tensors, stored dtype)."""
        for part in self.parts():
            part.load(tensors, self.rt)
        self.rt._shared.clear()
        self.loaded = True
        return self

    # --------------------------------------------------------------- builders
    @classmethod
    def load(cls, folder: str, dtype: Union[str, torch.dtype] = "bfloat16",
             device: Union[str, torch.device] = "cuda") -> "Model":
        raw = read_config_json(folder)
        arch = find_architecture(raw)
        config = arch.read_config(raw)
        model = cls(arch.plan(config), Runtime(torch.device(device), compute_dtype(dtype)), config)
        with TensorSource(folder) as source:
            # views of the mapped files: every tensor goes from the file's pages to the
            # device in one copy (parts that fuse or convert make their own host copy)
            tensors = bind(source, model.weight_specs(), where=folder, ignore=arch.ignore, copy=False)
            model.load_tensors(tensors)
            del tensors
        return model

    @classmethod
    def random(cls, config_json: Any, seed: int = 0, dtype: Union[str, torch.dtype] = "bfloat16",
               device: Union[str, torch.device] = "cuda", std: Optional[float] = None,
               norm_std: float = 0.0) -> "Model":
        """A model with random weights drawn on the device, without a folder
        (for measurements at sizes one would not write to disk)."""
        if hasattr(config_json, "to_json"):
            config_json = config_json.to_json()
        arch = find_architecture(config_json)
        config = arch.read_config(config_json)
        dt = compute_dtype(dtype)
        model = cls(arch.plan(config), Runtime(torch.device(device), dt), config)
        return model.load_tensors(random_tensors(model.weight_specs(), seed, std, norm_std, dt,
                                                 device=str(model.rt.device)))

    # ------------------------------------------------------------------ cache
    def new_cache(self, max_tokens: int, max_slots: Optional[int] = None) -> Cache:
        """A cache for up to `max_tokens` tokens held by live sequences, each
        sequence's count rounded up to a multiple of 64."""
        requests, shared = [], []
        for i, entry in enumerate(self.plan.schedule):
            if entry.cache is None:
                requests.append(list(self.blocks[entry.layer].cache_requests()))
                shared.append(None)
            else:
                requests.append([])
                shared.append(entry.cache)
        return Cache(requests, shared, max_tokens=max_tokens, max_slots=max_slots,
                     max_position=self.plan.max_position, dtype=self.rt.dtype, device=self.rt.device)

    def generate(self, prompts, max_new_tokens=50, **options):
        """Generate for a list of prompts (token ids); see engine/generate.py."""
        from .generate import generate
        return generate(self, prompts, max_new_tokens, **options)

    def weight_bytes(self) -> int:
        """Bytes of device memory the parts' weights hold (shared tables once)."""
        seen, total = set(), 0
        for part in self.parts():
            for v in vars(part).values():
                if isinstance(v, torch.Tensor) and v.data_ptr() not in seen:
                    seen.add(v.data_ptr())
                    total += v.numel() * v.element_size()
        return total
