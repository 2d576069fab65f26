"""Mixture of experts: every token runs through a few of many small gated feed-forwards.

    z = W_router x (float32) ,  s = softmax(z) over ALL router outputs
    chosen: the `top` largest of s + correction, taken only inside the `keep` best of `groups` equal groups
            of neighbouring outputs (a group's score is its largest s + correction)
    out = sum over chosen e of s_e * expert_e(x) ,  expert_e(x) = W_down_e (silu(W_gate_e x) * (W_up_e x))
    the last `identity` router outputs have no weights: their "expert" returns x itself

The weights are the plain scores (without the correction, not renormalized).  The router's product
and the choice are float32 in both engines.

With `router: "table"` there is no router product at all: an integer table [vocab, top] names the experts of
every token ID (no expert twice in a row), and each of them counts 1 / top.

How it runs: all experts' gate/up matrices are one matrix [E * 2F, d] (rows interleaved as in the dense
gated feed-forward, so the product's epilogue applies silu(gate) * up) and all down matrices one matrix
[d, E * F].  The routing kernel leaves a dense float32 weight per (token, expert), zero where the expert
was not chosen; the activations are scaled by it, and the ONE down product then sums the chosen experts'
outputs by itself.  The identity experts' share, x times the sum of their weights, is one more slab of
the branch's partial sums.  Nothing is read back and no shape depends on the choice, so decode steps are
recorded into graphs like any other; the price is that every expert is computed for every token, which
costs nothing while a step streams the weights anyway (decoding) and E / top times the needed products
for long prompt portions.
Tensors: `<name>router`, `correction` (or `table`), `e<i>.gate`, `e<i>.up`, `e<i>.down`.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..kernels import ops
from .base import Branch, ParamSpec, Part, register_part
from .linear import Linear


class RoutedFeedForward(Part):
    # Steps of a model with this part launch their kernels strictly one after the other.  With programmatic
    # dependent launch a 2,048-token FIRST step of a process at real widths (eight experts of 2,048 x 1,024)
    # never came back in about one run in five; it always did with the attribute off, and so did the same
    # model with dense feed-forwards.  Every wait in the kernels involved is bounded, and which of them stalls
    # was not found, so the overlap between consecutive kernels is given up for these models.
    serial_launches = True

    def __init__(self, spec, name):
        super().__init__(spec, name)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.inter = int(p["intermediate_size"])             # of one expert
        self.experts = int(p["num_experts"])
        self.identity = int(p.get("num_identity", 0))
        self.top = int(p["top"])
        self.groups = int(p.get("groups", 1))
        self.keep = int(p.get("keep_groups", self.groups))
        self.correction_tensor = bool(p.get("correction", True))
        self.routing = str(p.get("router", "scores"))         # "scores": a router product; "table": by token id
        if self.routing not in ("scores", "table"):
            raise ValueError(f"router {self.routing!r} is neither 'scores' nor 'table'")
        self.vocab = int(p.get("vocab_size", 0))
        if self.routing == "table" and (self.identity or self.vocab < 1):
            raise ValueError("a routing table needs the vocabulary's size and takes no identity experts")
        self.E = self.experts + self.identity
        if self.experts < 1 or self.identity < 0:
            raise ValueError(f"{self.experts} experts and {self.identity} identity experts")
        if self.E % self.groups or not 1 <= self.keep <= self.groups:
            raise ValueError(f"{self.E} router outputs in {self.groups} groups of which {self.keep} stay")
        if not 1 <= self.top <= self.keep * (self.E // self.groups):
            raise ValueError(f"{self.top} choices among {self.keep * (self.E // self.groups)} open experts")
        self.router = self.correction = self.table = None
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        n = self.name
        if self.routing == "table":
            out = {n + "table": ParamSpec((self.vocab, self.top), role="int", init="distinct", bounds=(0, self.experts))}
        else:
            out = {n + "router": ParamSpec((self.E, self.hidden), role="gain", init="normal")}
        if self.correction_tensor and self.routing == "scores":
            out[n + "correction"] = ParamSpec((self.E,), role="gain", init="normal")
        for e in range(self.experts):
            out[f"{n}e{e}.gate"] = ParamSpec((self.inter, self.hidden))
            out[f"{n}e{e}.up"] = ParamSpec((self.inter, self.hidden))
            out[f"{n}e{e}.down"] = ParamSpec((self.hidden, self.inter))
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        n, F, d = self.name, self.inter, self.hidden
        if self.routing == "table":
            self.table = tensors[n + "table"]
            lo, hi = int(self.table.min()), int(self.table.max())
            if lo < 0 or hi >= self.experts:
                raise ValueError(f"{n}table names experts {lo}..{hi}; there are {self.experts}")
        else:
            self.router = tensors[n + "router"]              # float32: the router's product is never rounded
            self.correction = tensors[n + "correction"] if self.correction_tensor else None
        rows = [torch.stack([tensors[f"{n}e{e}.gate"], tensors[f"{n}e{e}.up"]], dim=1).reshape(2 * F, d)
                for e in range(self.experts)]
        self.gate_up = Linear(torch.cat(rows, dim=0))
        self.down = Linear(torch.cat([tensors[f"{n}e{e}.down"] for e in range(self.experts)], dim=1))

    def streamed_weights(self):
        return [self.gate_up.weight, self.down.weight]

    def route(self, ctx, x: torch.Tensor):
        """float32 weights [N, E] (zero where an output was not chosen), ids int32 and weights float32 [N, top]."""
        N = x.shape[0]
        take = ctx.buffers.take
        if self.routing == "table":
            weights = take("moe_weights", N, (self.E,), torch.float32)
            ops.moe_table(weights, ctx.token_ids, self.table, ctx.token_feedback)
            return weights, None, None
        logits = take("moe_logits", N, (self.E,), torch.float32)
        ops.moe_logits(logits, x, self.router)
        weights = take("moe_weights", N, (self.E,), torch.float32)
        ids = take("moe_ids", N, (self.top,), torch.int32)
        picked = take("moe_picked", N, (self.top,), torch.float32)
        ops.moe_route(logits, self.correction, weights, ids, picked, self.groups, self.keep, self.top)
        return weights, ids, picked

    def forward(self, ctx, x: torch.Tensor) -> Branch:
        N, d, width = x.shape[0], self.hidden, self.experts * self.inter
        weights, _, _ = self.route(ctx, x)
        if ctx.can_fuse_silu_mul(N, self.gate_up.weight, x.dtype):
            act = self.gate_up(ctx, x, "moe_act", epilogue=1)
        else:
            gu = self.gate_up(ctx, x, "moe_gate_up")
            act = ctx.buffers.take("moe_act", N, (width,), ctx.dtype)
            ops.silu_mul(act, gu, interleaved=True)
        ops.moe_scale(act, weights, self.experts)
        S = ctx.gemm_splits(N, self.down.weight, act.dtype)
        slabs = S + (1 if self.identity else 0)
        partial = ctx.buffers.take_flat("branch", slabs * N * d, torch.float32).view(slabs, N, d)
        ctx.gemm(partial[:S], act, self.down.weight)
        if self.identity:
            ops.moe_passthrough(partial[S], x, weights, self.experts)
        return Branch(partial)


register_part("feed_forward", "routed_experts", RoutedFeedForward)
