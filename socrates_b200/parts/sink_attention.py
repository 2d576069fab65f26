"""Grouped-query softmax attention whose denominator holds one more term (a sink), with per-head
QK-RMSNorm, rotation, keys and values of different sizes, and an output gate.

    q, k, v = W_q x, W_k x, W_v x            H query heads and G key/value heads; q, k of `key_dim`, v of `value_dim`
    q, k = rotate(rmsnorm(q) * w_q), rotate(rmsnorm(k) * w_k)        (norm per head, gains shared by the heads)
    s_ij = (q_i . k_j) * scale,  j <= i  (and i - j < window, if one is given)
    p_ij = exp(s_ij) / (exp(sink) + sum_j exp(s_ij))                 (sink 0: "one added to the denominator")
    o_i = sum_j p_ij v_j ;  out = W_o (concat_h(o_i) * sigmoid(W_g x_i))

The gate is one value per head and value dim ("dim") or one per head ("head"), read from the same
input as the projections.  Scores, weights and the weighted sum are float32 (the CUDA-core attention
kernels; prompt portions in the bfloat16 engine with keys and values of one size of 64 or 128 run on the
tensor-core tile kernel, whose weights are two bfloat16 terms); keys are stored normed and rotated, so a layer with `own_kv: False` (its run reads an
earlier run's cache) has no k, v or k-norm tensors and brings only its queries, mask and gate.
All projections of a layer are one matrix product.
Tensors: `<name>q`, `k`, `v`, `q.norm`, `k.norm`, `g`, `o`.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..cache.manager import CacheNeeds, PagedKVSpec
from ..kernels import ops
from .base import Branch, ParamSpec, Part, build_part, register_part
from .linear import Linear


class GatedSinkAttention(Part):
    out_buffer = "branch"

    def __init__(self, spec, name):
        super().__init__(spec, name)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.H, self.G = int(p["num_heads"]), int(p["num_kv_heads"])
        self.dk, self.dv = int(p["key_dim"]), int(p["value_dim"])
        self.scale = float(p["scale"])
        self.qk_norm_eps = p.get("qk_norm_eps")                  # None: q and k are not normed
        self.sink: Optional[float] = p.get("sink")               # None: a plain softmax
        self.gate: Optional[str] = p.get("gate", "dim")
        self.window: Optional[int] = p.get("window")
        self.own_kv = bool(p.get("own_kv", True))
        self.position = build_part("position", p["position"], "")
        if self.H % self.G:
            raise ValueError(f"{self.H} query heads are no multiple of {self.G} key/value heads")
        if self.gate not in (None, "dim", "head"):
            raise ValueError(f"gate {self.gate!r} is neither 'dim', 'head' nor None")
        if not (1 <= self.dk <= 256 and 1 <= self.dv <= 256):
            raise ValueError(f"head sizes {self.dk} (keys) and {self.dv} (values) must be between 1 and 256")
        self.Cq = self.H * self.dk
        self.Ckv = self.G * (self.dk + self.dv) if self.own_kv else 0
        self.Cg = {None: 0, "dim": self.H * self.dv, "head": self.H}[self.gate]
        self.proj: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.q_gain = self.k_gain = None

    def parameters(self) -> Dict[str, ParamSpec]:
        n = self.name
        out = {n + "q": ParamSpec((self.Cq, self.hidden)), n + "o": ParamSpec((self.hidden, self.H * self.dv))}
        if self.own_kv:
            out[n + "k"] = ParamSpec((self.G * self.dk, self.hidden))
            out[n + "v"] = ParamSpec((self.G * self.dv, self.hidden))
        if self.qk_norm_eps is not None:
            out[n + "q.norm"] = ParamSpec((self.dk,), role="gain", init="gain")
            if self.own_kv:
                out[n + "k.norm"] = ParamSpec((self.dk,), role="gain", init="gain")
        if self.gate is not None:
            out[n + "g"] = ParamSpec((self.Cg, self.hidden))
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        n = self.name
        names = ["q", *(["k", "v"] if self.own_kv else []), *(["g"] if self.gate is not None else [])]
        self.proj = Linear(torch.cat([tensors[n + x] for x in names], dim=0))
        self.o = Linear(tensors[n + "o"])
        self.position.tables(self.o.weight.device)      # made now: no copy from the host inside a step
        if self.qk_norm_eps is not None:
            self.q_gain = tensors[n + "q.norm"]
            self.k_gain = tensors[n + "k.norm"] if self.own_kv else None

    def cache_needs(self) -> Optional[CacheNeeds]:
        if not self.own_kv:
            return None
        return CacheNeeds(paged=PagedKVSpec(self.G, self.dk, self.window, None if self.dv == self.dk else self.dv))

    def streamed_weights(self):
        return [self.proj.weight, self.o.weight]

    def partitions(self, ctx, N: int, max_len: int) -> int:
        """Into how many shares each token's visible keys are cut when every token is a block of its own: with
        few tokens (a decode step) the keys are shared out over about four blocks an SM, at least 64 keys a
        share, at most 16 shares.  A function of the token count and of limits alone (a recorded graph stays
        valid); it changes the order of additions, nothing else."""
        span = min(self.window or max_len, max_len)
        blocks = max(1, N * self.G)
        return max(1, min(16, (4 * ctx.num_sms) // blocks, -(-span // 64)))

    def forward(self, ctx, x: torch.Tensor, cache) -> Branch:
        if cache.writes != self.own_kv:
            raise ValueError(f"{self.name}: the plan and the part disagree on whose keys and values this layer uses")
        N = x.shape[0]
        proj = self.proj(ctx, x, "sa_proj")
        q = ctx.buffers.take("sa_q", N, (self.Cq,), ctx.dtype)
        k_pool, v_pool = cache.pools()
        table = cache.block_table()
        inv_freq, rotary_dim = self.position.tables(x.device)
        ops.qk_norm_rope_kvwrite(
            proj, q, k_pool if self.own_kv else None, v_pool if self.own_kv else None, self.q_gain, self.k_gain,
            inv_freq, rotary_dim, ctx.positions, ctx.token_rows, table,
            self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, self.H, self.G, self.dk,
            value_dim=self.dv, row_width=proj.shape[1], neighbours=self.position.neighbours,
            magnitude=getattr(self.position, "magnitude", 1.0))
        attn = ctx.buffers.take("sa_attn", N, (self.H * self.dv,), ctx.dtype)
        gate = proj[:, self.Cq + self.Ckv:] if self.gate is not None else None
        per_dim = self.gate == "dim"
        if (not ctx.all_decode and ctx.dtype == torch.bfloat16 and ctx.status is not None and self.dk == self.dv
                and ops.attention_tcgen05_supports(self.H, self.G, self.dk, k_pool.shape[2])):
            # prompt portions in the bfloat16 engine, keys and values of one size: the tensor-core tile kernel.
            # Scores are float32 sums of the bfloat16 q and k that the cache holds anyway; softmax is float32;
            # each weight enters the value product as two bfloat16 terms (16 bits of mantissa).
            ops.attention_prefill_tcgen05(attn, q, k_pool, v_pool, table, ctx.seq_starts, ctx.seq_rows,
                                          ctx.seq_first_pos, self.H, self.scale, ctx.status, self.window or 0,
                                          gate=gate, gate_per_dim=per_dim, sink=self.sink)
        elif (not ctx.all_decode and N >= 4 * ctx.num_seqs
                and ops.attention_bias_tile_supports(self.H, self.G, self.dk, self.dv, ctx.dtype)):
            # prompt portions: a tile of a request's consecutive tokens per block shares the keys it reads
            ops.attention_bias_tile(attn, q, k_pool, v_pool, table, ctx.seq_starts, ctx.seq_rows, ctx.seq_first_pos,
                                    self.H, self.scale, self.window or 0, gate=gate, gate_per_dim=per_dim,
                                    sink=self.sink)
        else:
            NP, part_o, part_ml = self.partitions(ctx, N, cache.manager.max_len), None, None
            if NP > 1:
                part_o = ctx.buffers.take_flat("attn_part_o", N * self.H * NP * self.dv, torch.float32)
                part_ml = ctx.buffers.take_flat("attn_part_ml", N * self.H * NP * 2, torch.float32)
            ops.attention_bias(attn, q, k_pool, v_pool, table, ctx.token_rows, ctx.positions, self.H, self.scale,
                               self.window or 0, gate=gate, num_partitions=NP, part_o=part_o, part_ml=part_ml,
                               gate_per_dim=per_dim, sink=self.sink)
        return Branch(self.o(ctx, attn, self.out_buffer, out="partial"))


register_part("mixer", "gated_sink_attention", GatedSinkAttention)
