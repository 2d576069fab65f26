"""SwiGLU feed-forward: down(up(x) * silu(gate(x))), no bias
(model/qwen/qwen_kv_cont.py:250-266).  gate and up are one matrix product here: when the
weights are bound their rows are interleaved (row 2f = gate_f, row 2f+1 = up_f), so that a
gate and its up value are neighbours in the product's output.  For many rows the
tensor-core kernel then applies SiLU*mul in its epilogue and the [N, 2F] intermediate is
never written; otherwise a SiLU*mul kernel reads the interleaved product.
silu(z) = z * sigmoid(z) in float32."""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..kernels import ops
from .base import Branch, ParamSpec, Part, register_part
from .linear import Linear


class SwiGLU(Part):
    def __init__(self, spec, name):
        super().__init__(spec, name)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        # tensor names after the part's prefix: gate, up, down (a plan may rename them)
        self.names = tuple(spec.params.get("names", ("gate_proj.weight", "up_proj.weight", "down_proj.weight")))
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        n = self.name
        return {
            n + self.names[0]: ParamSpec((self.inter, self.hidden)),
            n + self.names[1]: ParamSpec((self.inter, self.hidden)),
            n + self.names[2]: ParamSpec((self.hidden, self.inter)),
        }

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        n = self.name
        gate, up = tensors[n + self.names[0]], tensors[n + self.names[1]]
        self.gate_up = Linear(torch.stack([gate, up], dim=1).reshape(2 * self.inter, self.hidden))
        self.down = Linear(tensors[n + self.names[2]])

    def streamed_weights(self):
        """The weight matrices in the order in which forward() reads them."""
        return [self.gate_up.weight, self.down.weight]

    def forward(self, ctx, x: torch.Tensor) -> Branch:
        N = x.shape[0]
        if ctx.can_fuse_silu_mul(N, self.gate_up.weight, x.dtype):
            act = self.gate_up(ctx, x, "act", epilogue=1)
        else:
            gu = self.gate_up(ctx, x, "gate_up")
            act = ctx.buffers.take("act", N, (self.inter,), ctx.dtype)
            ops.silu_mul(act, gu, interleaved=True)
        return Branch(self.down(ctx, act, "branch", out="partial"))


register_part("feed_forward", "swiglu", SwiGLU)


class DenseFF(Part):
    """Two matrices with biases around one activation: down(act(up(x) + b_up)) + b_down.
    `activation`: "relu_squared" (max(z, 0)^2), "gelu_tanh" or "silu", computed in float32.
    Tensors: `<name>up`, `<name>up.b`, `<name>down`, `<name>down.b` (the suffixes can be
    renamed through the spec).  The up bias and the activation are one kernel that reads the
    product (its split-K partial sums where it was cut); the down bias travels with the
    branch and is added when the branch is folded into the residual."""

    def __init__(self, spec, name):
        super().__init__(spec, name)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.activation = str(spec.params.get("activation", "relu_squared"))
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"unknown activation {self.activation!r}; known: {sorted(ops.ACTIVATIONS)}")
        self.bias = bool(spec.params.get("bias", True))
        self.up: Optional[Linear] = None
        self.down: Optional[Linear] = None
        self.up_bias = self.down_bias = None

    def parameters(self) -> Dict[str, ParamSpec]:
        n = self.name
        out = {n + "up": ParamSpec((self.inter, self.hidden)), n + "down": ParamSpec((self.hidden, self.inter))}
        if self.bias:
            out[n + "up.b"] = ParamSpec((self.inter,), role="gain", init="normal")
            out[n + "down.b"] = ParamSpec((self.hidden,), role="gain", init="normal")
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        n = self.name
        self.up, self.down = Linear(tensors[n + "up"]), Linear(tensors[n + "down"])
        if self.bias:
            self.up_bias, self.down_bias = tensors[n + "up.b"], tensors[n + "down.b"]

    def streamed_weights(self):
        return [self.up.weight, self.down.weight]

    def forward(self, ctx, x: torch.Tensor) -> Branch:
        N = x.shape[0]
        u = self.up(ctx, x, "ff_up", out="model_or_partial")
        act = ctx.buffers.take("act", N, (self.inter,), ctx.dtype)
        ops.bias_act(act, u, self.up_bias, self.activation)
        return Branch(self.down(ctx, act, "branch", out="partial"), bias=self.down_bias)


register_part("feed_forward", "dense_act", DenseFF)


class ClampedGLU(Part):
    """A gated feed-forward whose gate and value are clamped, with biases on all three matrices:
        g = min(W_gate x + b_gate, limit) ,  u = clamp(W_up x + b_up, -limit, limit)
        out = W_down (g * sigmoid(alpha * g) * (u + offset)) + b_down
    `limit`, `alpha` and `offset` come from the spec.  gate and up are one matrix product (gate rows first);
    biases, clamps and the activation are one float32 kernel that reads the product (its split-K partial sums
    where it was cut); the down bias travels with the branch.  Tensors: `<name>gate`, `gate.b`, `up`, `up.b`,
    `down`, `down.b`."""

    def __init__(self, spec, name):
        super().__init__(spec, name)
        p = spec.params
        self.hidden, self.inter = int(p["hidden_size"]), int(p["intermediate_size"])
        self.limit, self.alpha, self.offset = float(p["limit"]), float(p.get("alpha", 1.702)), float(p.get("offset", 1.0))
        if not self.limit > 0:
            raise ValueError(f"a clamp at {self.limit}")
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None
        self.b_gate = self.b_up = self.b_down = None

    def parameters(self) -> Dict[str, ParamSpec]:
        n = self.name
        return {
            n + "gate": ParamSpec((self.inter, self.hidden)), n + "up": ParamSpec((self.inter, self.hidden)),
            n + "down": ParamSpec((self.hidden, self.inter)),
            n + "gate.b": ParamSpec((self.inter,), role="gain", init="around_zero"),
            n + "up.b": ParamSpec((self.inter,), role="gain", init="around_zero"),
            n + "down.b": ParamSpec((self.hidden,), role="gain", init="normal"),
        }

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        n = self.name
        self.gate_up = Linear(torch.cat([tensors[n + "gate"], tensors[n + "up"]], dim=0))
        self.down = Linear(tensors[n + "down"])
        self.b_gate, self.b_up, self.b_down = tensors[n + "gate.b"], tensors[n + "up.b"], tensors[n + "down.b"]

    def streamed_weights(self):
        return [self.gate_up.weight, self.down.weight]

    def forward(self, ctx, x: torch.Tensor) -> Branch:
        N = x.shape[0]
        gu = self.gate_up(ctx, x, "gate_up", out="model_or_partial")
        act = ctx.buffers.take("act", N, (self.inter,), ctx.dtype)
        ops.glu_clamp(act, gu, self.b_gate, self.b_up, self.limit, self.alpha, self.offset)
        return Branch(self.down(ctx, act, "branch", out="partial"), bias=self.b_down)


register_part("feed_forward", "clamped_glu", ClampedGLU)
