"""Grouped-query softmax attention whose scores are mixed across the heads before the softmax, with a
sigmoid gate on the concatenated heads.

    q, k, v = W_q x, W_k x, W_v x          H query heads and G key/value heads; q, k of `key_dim`, v of `value_dim`
    q, k = rotate(q), rotate(k)            (any position part; keys are stored rotated)
    r_g(i, j) = q_g(i) . k_kv(g)(j)        kv(g) = g / (H / G)
    s_h(i, j) = scale * sum_g talk[h, g] r_g(i, j)         (tensor `talk` [H, H]; the scale may sit on either side)
    keys j <= i (and i - j < window, if one is given); an ordinary softmax over them
    out = W_o (concat_h(softmax(s_h) v_kv(h)) * sigmoid(W_g x))        (`gate`: False leaves the gate out)

Scores, the mixing, weights and the weighted sum are float32 (`csrc/attention_talk.cu`): a block serves all
heads of a tile of a request's consecutive tokens, since every head's score reads every head's raw score;
a decode step gives each token a tile of its own and cuts its keys into shares.  All projections are one
matrix product.  Tensors: `<name>q`, `k`, `v`, `talk`, `g`, `o`.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..cache.manager import CacheNeeds, PagedKVSpec
from ..kernels import ops
from .base import Branch, ParamSpec, Part, build_part, register_part
from .linear import Linear


class TalkingAttention(Part):
    out_buffer = "branch"
    shared_projection = True       # a mixer that holds this one may make the projections (they must start its rows)

    def __init__(self, spec, name):
        super().__init__(spec, name)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.H, self.G = int(p["num_heads"]), int(p["num_kv_heads"])
        self.dk, self.dv = int(p["key_dim"]), int(p["value_dim"])
        self.scale = float(p["scale"])
        self.gate = bool(p.get("gate", True))
        self.window: Optional[int] = p.get("window")
        self.position = build_part("position", p["position"], "")
        if self.H % self.G:
            raise ValueError(f"{self.H} query heads are no multiple of {self.G} key/value heads")
        if not (1 <= self.dk <= 256 and 1 <= self.dv <= 256):
            raise ValueError(f"head sizes {self.dk} (keys) and {self.dv} (values) must be between 1 and 256")
        self.Cq, self.Ckv = self.H * self.dk, self.G * (self.dk + self.dv)
        self.Cg = self.H * self.dv if self.gate else 0
        self.proj: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.talk = None

    def parameters(self) -> Dict[str, ParamSpec]:
        n = self.name
        out = {n + "q": ParamSpec((self.Cq, self.hidden)), n + "k": ParamSpec((self.G * self.dk, self.hidden)),
               n + "v": ParamSpec((self.G * self.dv, self.hidden)), n + "o": ParamSpec((self.hidden, self.H * self.dv)),
               n + "talk": ParamSpec((self.H, self.H), role="gain", init="uniform", bounds=(-0.5, 1.0))}
        if self.gate:
            out[n + "g"] = ParamSpec((self.Cg, self.hidden))
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        n = self.name
        names = ["q", "k", "v", *(["g"] if self.gate else [])]
        self.proj = Linear(torch.cat([tensors[n + x] for x in names], dim=0))
        self.o = Linear(tensors[n + "o"])
        self.talk = tensors[n + "talk"]
        self.position.tables(self.o.weight.device)      # made now: no copy from the host inside a step

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(paged=PagedKVSpec(self.G, self.dk, self.window, None if self.dv == self.dk else self.dv))

    def streamed_weights(self):
        return [*([self.proj.weight] if self.proj is not None else []), self.o.weight]

    def partitions(self, ctx, N: int, max_len: int) -> int:
        """Into how many shares a decode step cuts each token's keys: about two blocks an SM, at least 128 keys a
        share, at most 32 shares.  A function of the token count and of limits alone (a recorded graph stays
        valid); it changes the order of additions, nothing else."""
        span = min(self.window or max_len, max_len)
        return max(1, min(32, (2 * ctx.num_sms) // max(1, N), -(-span // 128)))

    def forward(self, ctx, x: torch.Tensor, cache, proj=None) -> Branch:
        N = x.shape[0]
        if proj is None:
            proj = self.proj(ctx, x, "ta_proj")
        else:
            proj, first = proj                   # a wider product made outside; this mixer's columns come first
            if first != 0:
                raise ValueError("the rotation kernel reads its heads from the start of a row")
        q = ctx.buffers.take("ta_q", N, (self.Cq,), ctx.dtype)
        k_pool, v_pool = cache.pools()
        table = cache.block_table()
        inv_freq, rotary_dim = self.position.tables(x.device)
        ops.qk_norm_rope_kvwrite(
            proj, q, k_pool, v_pool, None, None, inv_freq, rotary_dim, ctx.positions, ctx.token_rows, table, 0.0,
            self.H, self.G, self.dk, value_dim=self.dv, row_width=proj.shape[1],
            neighbours=self.position.neighbours, magnitude=getattr(self.position, "magnitude", 1.0))
        attn = ctx.buffers.take("ta_attn", N, (self.H * self.dv,), ctx.dtype)
        gate = proj[:, self.Cq + self.Ckv:self.Cq + self.Ckv + self.Cg] if self.gate else None
        if ctx.all_decode:
            NP, part_o, part_ml = self.partitions(ctx, N, cache.manager.max_len), None, None
            if NP > 1:
                part_o = ctx.buffers.take_flat("attn_part_o", N * self.H * NP * self.dv, torch.float32)
                part_ml = ctx.buffers.take_flat("attn_part_ml", N * self.H * NP * 2, torch.float32)
            ops.attention_talk(attn, q, k_pool, v_pool, table, ctx.seq_starts, ctx.seq_rows, ctx.seq_first_pos,
                               self.talk, self.H, self.scale, self.window or 0, gate=gate, queries_per_tile=1,
                               num_partitions=NP, part_o=part_o, part_ml=part_ml)
        else:
            ops.attention_talk(attn, q, k_pool, v_pool, table, ctx.seq_starts, ctx.seq_rows, ctx.seq_first_pos,
                               self.talk, self.H, self.scale, self.window or 0, gate=gate)
        return Branch(self.o(ctx, attn, self.out_buffer, out="partial"))


register_part("mixer", "talking_attention", TalkingAttention)
