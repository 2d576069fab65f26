"""Two recurrent mixers whose gates read only the current token.

"min_gru": one state value per channel of `width`:
    z = sigmoid(W_z x + b_z) ,  u = W_x x + b_x ,  c = u + 1/2 where u >= 0, sigmoid(u) where u < 0
    S_t = (1 - z) S_(t-1) + z c ;  out = W_o (S_t * silu(W_g x))
Tensors: `<name>z`, `z.b`, `x`, `x.b`, `g`, `o`.

"gated_linear_attention": a matrix state per head in which the forget gate also decides what is written:
    q = silu(W_q x)  (H heads of `key_dim`) ,  v = W_v x  (H heads of `value_dim`)
    f = l + (1 - l) sigmoid(W_f x + b_f)      per head and key channel, l the lower bound (tensor `lower`)
    S_t = diag(f) S_(t-1) + (1 - f) v^T ;  o = S_t^T q
    out = W_o concat_h(o / sqrt(mean(o^2) + eps) * w)          (one gain of `value_dim`, shared by the heads)
Tensors: `<name>q`, `f`, `f.b`, `lower`, `v`, `norm`, `o`.

The states are float32 and live in the request's state slot, so prompts may arrive in portions and
requests decode side by side.  Gates, decays, the recurrences and the norm are float32 in both engines.
All projections of a mixer are one matrix product; the recurrence is one kernel that walks a request's
tokens with the state in registers (the head norm a small second one).
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..cache.manager import CacheNeeds, StateSpec
from ..kernels import ops
from .base import Branch, ParamSpec, Part, register_part
from .linear import Linear


class MinGRU(Part):
    out_buffer = "branch"

    def __init__(self, spec, name):
        super().__init__(spec, name)
        p = spec.params
        self.hidden, self.W = int(p["hidden_size"]), int(p["width"])
        self.bias = bool(p.get("bias", True))
        self.proj: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.bz = self.bx = None

    def parameters(self) -> Dict[str, ParamSpec]:
        n = self.name
        out = {n + x: ParamSpec((self.W, self.hidden)) for x in ("z", "x", "g")}
        out[n + "o"] = ParamSpec((self.hidden, self.W))
        if self.bias:
            out[n + "z.b"] = ParamSpec((self.W,), role="gain", init="around_zero")
            out[n + "x.b"] = ParamSpec((self.W,), role="gain", init="around_zero")
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        n = self.name
        self.proj = Linear(torch.cat([tensors[n + x] for x in ("z", "x", "g")], dim=0))
        self.o = Linear(tensors[n + "o"])
        if self.bias:
            self.bz, self.bx = tensors[n + "z.b"], tensors[n + "x.b"]

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(state={"S": StateSpec((self.W,), torch.float32)})

    def streamed_weights(self):
        return [self.proj.weight, self.o.weight]

    def forward(self, ctx, x: torch.Tensor, cache) -> Branch:
        N = x.shape[0]
        proj = self.proj(ctx, x, "gru_proj")
        y = ctx.buffers.take("gru_y", N, (self.W,), ctx.dtype)
        ops.min_gru(y, proj, self.bz, self.bx, cache.state("S"), ctx.seq_starts, ctx.seq_rows)
        return Branch(self.o(ctx, y, self.out_buffer, out="partial"))


register_part("mixer", "min_gru", MinGRU)


class GatedLinearAttention(Part):
    out_buffer = "branch"
    shared_projection = True       # a mixer that holds this one may make the projections

    def __init__(self, spec, name):
        super().__init__(spec, name)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.H, self.dk, self.dv = int(p["num_heads"]), int(p["key_dim"]), int(p["value_dim"])
        self.eps = float(p["norm_eps"])
        if not (1 <= self.dk <= 256 and self.dv >= 1):
            raise ValueError(f"head sizes {self.dk} (keys, at most 256) and {self.dv} (values)")
        self.Cqk, self.Cv = self.H * self.dk, self.H * self.dv
        self.proj: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.f_bias = self.lower = self.norm_w = None

    def parameters(self) -> Dict[str, ParamSpec]:
        n = self.name
        return {
            n + "q": ParamSpec((self.Cqk, self.hidden)), n + "f": ParamSpec((self.Cqk, self.hidden)),
            n + "v": ParamSpec((self.Cv, self.hidden)), n + "o": ParamSpec((self.hidden, self.Cv)),
            n + "f.b": ParamSpec((self.Cqk,), role="gain", init="uniform", bounds=(-1.0, 3.0)),
            n + "lower": ParamSpec((self.Cqk,), role="gain", init="uniform", bounds=(0.0, 0.9)),
            n + "norm": ParamSpec((self.dv,), role="gain", init="gain"),
        }

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        n = self.name
        self.proj = Linear(torch.cat([tensors[n + x] for x in ("q", "f", "v")], dim=0))
        self.o = Linear(tensors[n + "o"])
        self.f_bias, self.lower, self.norm_w = tensors[n + "f.b"], tensors[n + "lower"], tensors[n + "norm"]

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(state={"S": StateSpec((self.H, self.dk, self.dv), torch.float32)})

    def streamed_weights(self):
        return [*([self.proj.weight] if self.proj is not None else []), self.o.weight]

    def forward(self, ctx, x: torch.Tensor, cache, proj=None) -> Branch:
        N = x.shape[0]
        proj, c0 = (self.proj(ctx, x, "gla_proj"), 0) if proj is None else proj      # or columns of a wider product
        y = ctx.buffers.take("gla_y", N, (self.Cv,), ctx.dtype)
        raw = ctx.buffers.take("gla_raw", N, (self.Cv,), torch.float32)
        longest = N - ctx.num_seqs + 1                 # no request brings more: a function of the step's shape alone
        need = ops.gated_linear_attention_seg_scratch(ctx.num_seqs, longest, self.H, self.dk, self.dv)
        segs = ctx.buffers.take_flat("gla_segments", need, torch.float32) if need else None
        ops.gated_linear_attention(y, proj, (c0, c0 + self.Cqk, c0 + 2 * self.Cqk), self.f_bias, self.lower, self.norm_w,
                                   cache.state("S"), ctx.seq_starts, ctx.seq_rows, self.H, self.dk, self.dv,
                                   self.eps, scratch=raw, longest=longest, seg_scratch=segs)
        return Branch(self.o(ctx, y, self.out_buffer, out="partial"))


register_part("mixer", "gated_linear_attention", GatedLinearAttention)
