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
a decode step gives each token a tile of its own and cuts its keys into shares.  One exception, in the bfloat16
engine only: a step that is ONE long prompt portion runs both products on the tensor cores through the engine's
matrix product (`dense_form`): keys gathered out of their pages, raw scores of a block of queries as one product
per KV head (float32 sums over the bfloat16 q and k), mixing, mask and softmax in float32 by a kernel that writes
every weight as two bfloat16 terms, the weighted values as one more product over both terms.  All projections are
one matrix product.  Tensors: `<name>q`, `k`, `v`, `talk`, `g`, `o`.
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

    # Tokens from which a lone prompt portion takes the tensor-core form.  It pays from a few hundred tokens on; it
    # is kept to long portions because its chain of launches once did not come back (see dense_form).
    DENSE_FROM = 1536
    DENSE_SCORES = 1 << 27     # most raw scores of a block of queries (float32: 512 MB)

    def dense_form(self, ctx, q, gate, attn, k_pool, v_pool, table) -> bool:
        """The tensor-core form for a step that is one prompt portion of one request; False if the step is not
        such a step (the caller then runs the tile kernel)."""
        import os
        entries = ctx.host_batch
        N = q.shape[0]
        if (ctx.dtype != torch.bfloat16 or ctx.status is None or entries is None or len(entries) != 1
                or N < self.DENSE_FROM or self.dk % 8 or self.dv % 8 or self.H > 64 or self.dv > 256
                or os.environ.get("SOCRATES_TALK_DENSE", "1") == "0"):
            return False
        e = entries[0]
        start, row = int(e.start), int(e.row)
        C = start + N
        Cp = -(-C // 64) * 64
        if Cp * 4 > 200 * 1024:
            return False
        H, Hkv, G, dk, dv = self.H, self.G, self.H // self.G, self.dk, self.dv
        nb_most = max(64, min(N, self.DENSE_SCORES // (H * Cp)))
        take = ctx.buffers.take_flat
        Kc = take("talk_kc", Hkv * Cp * dk, ctx.dtype)
        Vt = take("talk_vt", Hkv * dv * 2 * Cp, ctx.dtype)
        Qg = take("talk_qg", H * nb_most * dk, ctx.dtype)
        S = take("talk_s", H * nb_most * Cp, torch.float32)
        P = take("talk_p", H * nb_most * 2 * Cp, ctx.dtype)
        O = take("talk_o", H * nb_most * dv, torch.float32)
        trow = table[row]
        args = (q, k_pool, v_pool, trow, Kc, Vt, Qg, S, P, O, attn, gate, self.talk, H)
        # these launches are plainly serial: a first 2,048-token step with them launched dependently never came back
        ops.set_dependent_launch(False)
        try:
            self._dense_steps(ctx, args, N, C, Cp, start, nb_most, S, Qg, Kc, O, P, Vt)
        finally:
            ops.set_dependent_launch(ctx.dependent_launch)
        return True

    def _dense_steps(self, ctx, args, N, C, Cp, start, nb_most, S, Qg, Kc, O, P, Vt) -> None:
        H, Hkv, G, dk, dv = self.H, self.G, self.H // self.G, self.dk, self.dv
        ops.attention_talk_dense_step(0, *args, C, Cp, 0, 1, start, self.window or 0, self.scale)
        for n0 in range(0, N, nb_most):
            nb = min(nb_most, N - n0)
            tail = (C, Cp, n0, nb, start + n0, self.window or 0, self.scale)
            ops.attention_talk_dense_step(1, *args, *tail)
            for kh in range(Hkv):
                ctx.gemm(S[kh * G * nb * Cp:(kh + 1) * G * nb * Cp].view(G * nb, Cp),
                         Qg[kh * G * nb * dk:(kh + 1) * G * nb * dk].view(G * nb, dk),
                         Kc[kh * Cp * dk:(kh + 1) * Cp * dk].view(Cp, dk))
            ops.attention_talk_dense_step(2, *args, *tail)
            for kh in range(Hkv):
                ctx.gemm(O[kh * G * nb * dv:(kh + 1) * G * nb * dv].view(G * nb, dv),
                         P[kh * G * nb * 2 * Cp:(kh + 1) * G * nb * 2 * Cp].view(G * nb, 2 * Cp),
                         Vt[kh * dv * 2 * Cp:(kh + 1) * dv * 2 * Cp].view(dv, 2 * Cp))
            ops.attention_talk_dense_step(3, *args, *tail)

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
        elif not self.dense_form(ctx, q, gate, attn, k_pool, v_pool, table):
            ops.attention_talk(attn, q, k_pool, v_pool, table, ctx.seq_starts, ctx.seq_rows, ctx.seq_first_pos,
                               self.talk, self.H, self.scale, self.window or 0, gate=gate)
        return Branch(self.o(ctx, attn, self.out_buffer, out="partial"))


register_part("mixer", "talking_attention", TalkingAttention)
