"""Token embedding and the output head.

Embedding: x = table[ids] (model/qwen/qwen_kv_paged.py:198,219), widened to the
float32 residual and multiplied by `scale` where the plan gives one.  Head: logits = x W^T with W the embedding table when the
configuration ties them (:224) or `lm_head.weight` otherwise; only the rows whose
logits were asked for are computed, in float32; with `softcap` c they become c * tanh(logits / c);
with `scale` they are multiplied by a constant.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..kernels import ops
from .base import ParamSpec, Part, ResidualStream, build_part, register_part
from .linear import Linear


class Embedding(Part):
    def __init__(self, spec, name):
        super().__init__(spec, name)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.tensor = self.name + str(spec.params.get("suffix", "weight"))
        self.scale = float(spec.params.get("scale", 1.0))      # the looked-up rows times a constant, in float32
        self.table: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        return {self.tensor: ParamSpec((self.vocab, self.hidden))}

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        self.table = tensors[self.tensor]

    def forward(self, ctx) -> torch.Tensor:
        out = ctx.buffers.take("residual", ctx.num_tokens, (self.hidden,), torch.float32)
        ops.embed(out, self.table, ctx.token_ids, ctx.token_feedback, self.scale)
        return out


class LMHead(Part):
    def __init__(self, spec, name):
        super().__init__(spec, name)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.tied_to: Optional[str] = spec.params.get("tied_to")
        self.tensor = self.name + str(spec.params.get("suffix", "weight"))
        cap = spec.params.get("softcap")                      # logits <- cap * tanh(logits / cap)
        self.softcap: Optional[float] = float(cap) if cap else None
        if self.softcap is not None and not self.softcap > 0:
            raise ValueError(f"a logit cap of {self.softcap}")
        self.scale = float(spec.params.get("scale", 1.0))      # logits <- logits * scale, in float32
        self.linear: Optional[Linear] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        if self.tied_to is not None:
            return {self.tied_to: ParamSpec((self.vocab, self.hidden))}
        return {self.tensor: ParamSpec((self.vocab, self.hidden))}

    def duplicates(self) -> Dict[str, str]:
        """A tied head reads the embedding; a file may still carry a copy under the head's name."""
        return {self.tensor: self.tied_to} if self.tied_to is not None else {}

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        self.linear = Linear(tensors[self.tied_to or self.tensor])

    def streamed_weights(self):
        return [self.linear.weight]

    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        logits = self.linear(ctx, x, "logits", out="wanted_float32")
        if self.scale != 1.0:
            ops.scale_(logits, self.scale)
        if self.softcap is not None:
            ops.softcap(logits, self.softcap)
        return logits


register_part("embedding", "embedding", Embedding)
register_part("head", "lm_head", LMHead)


class NormedEmbedding(Part):
    """x = norm(table[ids]): the looked-up rows are normed before they become the residual
    stream.  The norm is a part of its own kind (`norm` in the spec); its output is
    float32 in both engines, since it IS the residual."""

    def __init__(self, spec, name):
        super().__init__(spec, name)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.tensor = self.name + str(spec.params.get("suffix", "weight"))
        norm_spec = spec.params["norm"]
        self.norm = build_part("norm", norm_spec, self.name + norm_spec.name)
        self.table: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        return {self.tensor: ParamSpec((self.vocab, self.hidden)), **self.norm.parameters()}

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        self.table = tensors[self.tensor]
        self.norm.bind(tensors, dtype)

    def forward(self, ctx) -> torch.Tensor:
        raw = ctx.buffers.take("embedded", ctx.num_tokens, (self.hidden,), torch.float32)
        ops.embed(raw, self.table, ctx.token_ids, ctx.token_feedback)
        return self.norm.apply(ctx, ResidualStream(raw), buffer="residual", out_dtype=torch.float32)


register_part("embedding", "normed_embedding", NormedEmbedding)
