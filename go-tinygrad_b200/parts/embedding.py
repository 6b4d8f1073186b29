"""Token embedding and the output head.

``token_embedding``: x = E[token], unscaled (model/inference_helpers.go:9-34);
it starts the float32 residual stream.  Parameters: ``vocab_size``,
``hidden_size``, ``weight`` and optionally ``position`` (a position PartSpec
whose `on_embedding` hook acts on the embedded tokens).

``lm_head``: logits = x . LM^T in float32 for the rows it is given
(model/inference_helpers.go:122-148).  ``weight`` names the table; with
``tied`` it is the embedding's tensor and one device copy serves both
(model/llama.go:490-494 decides tying by the tensor's presence; here the
configuration's flag decides and a stray ``ignored`` tensor is tolerated).
"""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from ..kernels import ops
from ..weights.binder import WeightSpec
from .base import (Embedding, Head, ResidualStream, Runtime, StepContext, build_part,
                   register_part)


@register_part("embedding", "token_embedding")
class TokenEmbedding(Embedding):
    def __init__(self, spec):
        super().__init__(spec)
        self.vocab = int(self.param("vocab_size"))
        self.hidden = int(self.param("hidden_size"))
        self.weight_name = str(self.param("weight"))
        pos = self.p.get("position")
        self.position = build_part("position", pos) if pos is not None else None
        self.table: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.weight_name, (self.vocab, self.hidden), role="table")]

    def children(self):
        return [self.position] if self.position else []

    def load(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        self.table = rt.matrix(tensors[self.weight_name], share_as=self.weight_name)

    def forward(self, ctx: StepContext) -> ResidualStream:
        residual = ctx.rt.empty(ctx.n_tokens, self.hidden, dtype=torch.float32, lifetime="step")
        ops.embed(ctx.tokens, self.table, residual)
        stream = ResidualStream(residual)
        if self.position:
            self.position.on_embedding(stream, ctx)
        return stream


@register_part("head", "lm_head")
class LMHead(Head):
    def __init__(self, spec):
        super().__init__(spec)
        self.vocab = int(self.param("vocab_size"))
        self.hidden = int(self.param("hidden_size"))
        self.weight_name = str(self.param("weight"))
        self.tied = bool(self.p.get("tied", False))
        self.ignored = self.p.get("ignored")
        self.table: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        specs = [WeightSpec(self.weight_name, (self.vocab, self.hidden), role="table")]
        if self.ignored:
            specs.append(WeightSpec(str(self.ignored), (self.vocab, self.hidden), role="ignored",
                                    optional=True))
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        self.table = rt.matrix(tensors[self.weight_name], share_as=self.weight_name)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        logits = ctx.rt.result(x.shape[0], self.vocab, dtype=torch.float32)
        ops.linear(x, self.table, logits)
        return logits
