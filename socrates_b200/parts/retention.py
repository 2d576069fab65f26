"""Retention: linear attention with one fixed decay per head and no softmax.

For each head, with q_t, k_t of `key_dim` and v_t of `value_dim`:
    q_t, k_t = rotate(q_t), rotate(k_t) * key_scale         (the position part's table)
    S_t = decay_h * S_{t-1} + k_t v_t^T ,   o_t = S_t^T q_t
    y_t = unit_rms(o_t) * silu(g_t) ,       out_t = W_o concat_h(y_t)
There is no denominator; each head's output is divided by its root mean square instead.
The state S [heads, key_dim, value_dim] is float32 and lives in the request's state slot,
so prompts may arrive in portions and requests decode side by side.  q, k, v and g are one
matrix product (the weights are concatenated when they are bound); rotation, scaling, the
recurrence, the norm and the gate are one kernel that walks each request's tokens in order.
Tensors: `<name>q`, `k`, `v`, `g`, `o`.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..cache.manager import CacheNeeds, StateSpec
from ..kernels import ops
from .base import Branch, ParamSpec, Part, build_part, register_part
from .linear import Linear


class Retention(Part):
    out_buffer = "branch"

    def __init__(self, spec, name):
        super().__init__(spec, name)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.H = int(p["num_heads"])
        self.dk = int(p["key_dim"])
        self.dv = int(p["value_dim"])
        self.decay = [float(x) for x in p["decay"]]
        if len(self.decay) != self.H:
            raise ValueError(f"{len(self.decay)} decays for {self.H} heads")
        self.eps = float(p["norm_eps"])
        self.key_scale = float(p.get("key_scale", self.dk ** -0.5))
        self.position = build_part("position", p["position"], "")
        if getattr(self.position, "magnitude", 1.0) != 1.0:
            raise ValueError("the retention kernel rotates with plain cosines and sines; a scaled encoding is not served")
        self.qkvg: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.decay_t: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        n, H = self.name, self.H
        return {n + "q": ParamSpec((H * self.dk, self.hidden)), n + "k": ParamSpec((H * self.dk, self.hidden)),
                n + "v": ParamSpec((H * self.dv, self.hidden)), n + "g": ParamSpec((H * self.dv, self.hidden)),
                n + "o": ParamSpec((self.hidden, H * self.dv))}

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        n = self.name
        self.qkvg = Linear(torch.cat([tensors[n + x] for x in ("q", "k", "v", "g")], dim=0))
        self.o = Linear(tensors[n + "o"])
        self.decay_t = torch.tensor(self.decay, dtype=torch.float32, device=self.o.weight.device)
        self.position.tables(self.o.weight.device)      # made now: no copy from the host inside a step
        getattr(self.position, "low_table", lambda d: None)(self.o.weight.device)

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(state=StateSpec((self.H, self.dk, self.dv), torch.float32))

    def streamed_weights(self):
        return [self.qkvg.weight, self.o.weight]

    def forward(self, ctx, x: torch.Tensor, cache) -> Branch:
        N, H = x.shape[0], self.H
        qkvg = self.qkvg(ctx, x, "ret_qkvg")
        y = ctx.buffers.take("ret_y", N, (H * self.dv,), ctx.dtype)
        inv_freq, rotary_dim = self.position.tables(x.device)
        offsets = (0, H * self.dk, 2 * H * self.dk, 2 * H * self.dk + H * self.dv)
        scratch = None
        if not ctx.all_decode and ctx.num_seqs * H < ctx.num_sms:
            # few requests with long portions: scratch lets every chunk be a block of its own
            size = ops.retention_scratch_size(N, ctx.num_seqs, H, self.dk, self.dv)
            if 0 < size <= (1 << 28):
                scratch = ctx.buffers.take_flat("ret_scratch", size, torch.float32)
        ops.retention(y, qkvg, offsets, cache.state(), self.decay_t, inv_freq, rotary_dim, ctx.seq_starts,
                      ctx.seq_rows, ctx.seq_first_pos, self.eps, self.key_scale, chunked=not ctx.all_decode,
                      inv_freq_lo=getattr(self.position, "low_table", lambda d: None)(x.device), scratch=scratch)
        return Branch(self.o(ctx, y, self.out_buffer, out="partial"))


register_part("mixer", "retention", Retention)
