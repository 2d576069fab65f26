"""Differential attention: every query head carries two score maps over one set of values.

    q = W_q x + b_q   [H heads x (map 1 | map 2) x dim]      k = W_k x + b_k   [G heads x (map 1 | map 2) x dim]
    v = W_v x + b_v   [G heads x vdim]                        (query head h reads KV head h // (H / G))
    each map of q and k rotates its first `rotary_dim` dims (halves pairing; keys are stored rotated)
    s1 = (q1 . k1) * scale ,  s2 = (q2 . k2) * scale          over the keys j <= i that the mask leaves:
                                                               i - j < window, or j < keep_first (no window: all)
    o = softmax(s1) v - lambda * softmax(s2) v                lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff
    o <- o / sqrt(mean(o^2) + eps) * (1 - diff)               per head over its vdim values, no gain
    out = W_o concat_h(o)

`lambda` is one number for the layer, made once in float32 when the weights are bound.  The biases are
optional (`bias`).  Scores, softmax weights, weighted sums, the difference and the head norm are float32
in both engines (the CUDA-core kernels of `attention_diff.cu`); q, k and v are one matrix product, whose
bias is added by the rotation kernel; the cache holds key rows of 2 * dim dims and value rows of vdim.
Tensors: `<name>q`, `k`, `v` (each with `.b`), `lq1`, `lk1`, `lq2`, `lk2`, `o`.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..cache.manager import CacheNeeds, PagedKVSpec
from ..kernels import ops
from .base import Branch, ParamSpec, Part, build_part, register_part
from .linear import Linear


class DifferentialAttention(Part):
    def __init__(self, spec, name):
        super().__init__(spec, name)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.H, self.G = int(p["num_heads"]), int(p["num_kv_heads"])
        self.dim, self.dv = int(p["map_dim"]), int(p["value_dim"])
        self.scale = float(p["scale"])
        self.diff = float(p["diff"])
        self.eps = float(p["norm_eps"])
        self.window: Optional[int] = p.get("window")
        self.keep_first = int(p.get("keep_first", 0)) if self.window is not None else 0
        self.bias = bool(p.get("bias", True))
        self.position = build_part("position", p["position"], "")
        if self.H % self.G:
            raise ValueError(f"{self.H} query heads are no multiple of {self.G} key/value heads")
        if not (1 <= self.dim <= 128 and 1 <= self.dv <= 256):
            raise ValueError(f"maps of {self.dim} dims (1 to 128) and values of {self.dv} (1 to 256)")
        if self.window is not None and self.window < 1:
            raise ValueError(f"a window of {self.window} keys")
        if getattr(self.position, "neighbours", False):
            raise ValueError("the maps of a head rotate in halves")
        self.Cq, self.Ck, self.Cv = self.H * 2 * self.dim, self.G * 2 * self.dim, self.G * self.dv
        self.proj: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.proj_bias: Optional[torch.Tensor] = None
        self.lam: Optional[float] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        n = self.name
        out = {n + "q": ParamSpec((self.Cq, self.hidden)), n + "k": ParamSpec((self.Ck, self.hidden)),
               n + "v": ParamSpec((self.Cv, self.hidden)), n + "o": ParamSpec((self.hidden, self.H * self.dv))}
        if self.bias:
            for x, c in (("q", self.Cq), ("k", self.Ck), ("v", self.Cv)):
                out[f"{n}{x}.b"] = ParamSpec((c,), role="gain", init="normal")
        for x in ("lq1", "lk1", "lq2", "lk2"):
            out[n + x] = ParamSpec((self.dim,), role="gain", init="around_zero")
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        n = self.name
        self.proj = Linear(torch.cat([tensors[n + x] for x in ("q", "k", "v")], dim=0))
        self.o = Linear(tensors[n + "o"])
        if self.bias:
            self.proj_bias = torch.cat([tensors[f"{n}{x}.b"].float() for x in ("q", "k", "v")]).contiguous()
        t = lambda x: tensors[n + x].float()
        self.lam = float(torch.exp((t("lq1") * t("lk1")).sum()) - torch.exp((t("lq2") * t("lk2")).sum())) + self.diff
        self.position.tables(self.o.weight.device)      # made now: no copy from the host inside a step

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(paged=PagedKVSpec(self.G, 2 * self.dim, self.window,
                                            None if self.dv == 2 * self.dim else self.dv,
                                            keep_first=self.keep_first))

    def streamed_weights(self):
        return [self.proj.weight, self.o.weight]

    def partitions(self, ctx, N: int, max_len: int) -> int:
        """Into how many shares each token's visible keys are cut when every token is a block of its own: about
        four blocks an SM, at least 64 keys a share, at most 16 shares.  A function of the token count and of
        limits alone (a recorded graph stays valid); it changes the order of additions, nothing else."""
        span = max_len if self.window is None else min(self.window + self.keep_first, max_len)
        blocks = max(1, N * self.G)
        return max(1, min(16, (4 * ctx.num_sms) // blocks, -(-span // 64)))

    def forward(self, ctx, x: torch.Tensor, cache) -> Branch:
        N = x.shape[0]
        proj = self.proj(ctx, x, "da_proj", out="model_or_partial")
        k_pool, v_pool = cache.pools()
        table = cache.block_table()
        inv_freq, rotary_dim = self.position.tables(x.device)
        # Prompt portions in the bfloat16 engine, key rows and value heads of one size of 64 or 128: the tensor-core
        # tile kernel.  Every (head, map) is a query row of its own that holds its map's dims and zeros where the
        # other map's are, so the product with a whole key row is that map's score (adding zeros is exact); scores
        # are float32 sums over the bfloat16 q and k that the cache holds anyway, softmax is float32, each weight
        # enters the value product as two bfloat16 terms, and both maps' rows come back in float32 for the
        # difference and the head norm.
        tensor_cores = (not ctx.all_decode and N >= 4 * ctx.num_seqs and ctx.dtype == torch.bfloat16
                        and ctx.status is not None and 2 * self.dim == self.dv
                        and ops.attention_tcgen05_supports(2 * self.H, self.G, self.dv, k_pool.shape[2]))
        q = ctx.buffers.take("da_q", N, (self.Cq * (2 if tensor_cores else 1),), ctx.dtype)
        ops.qk_norm_rope_kvwrite(
            proj, q, k_pool if cache.writes else None, v_pool if cache.writes else None, None, None,
            inv_freq, rotary_dim, ctx.positions, ctx.token_rows, table, 0.0, self.H, self.G, 2 * self.dim,
            value_dim=self.dv, row_width=self.Cq + self.Ck + self.Cv, bias=self.proj_bias, map_dim=self.dim,
            magnitude=self.position.magnitude, spread_maps=tensor_cores)
        attn = ctx.buffers.take("da_attn", N, (self.H * self.dv,), ctx.dtype)
        window, out_scale = self.window or 0, 1.0 - self.diff
        if tensor_cores:
            maps = ctx.buffers.take("da_maps", N, (self.H * 2 * self.dv,), torch.float32)
            ops.attention_prefill_tcgen05(None, q, k_pool, v_pool, table, ctx.seq_starts, ctx.seq_rows,
                                          ctx.seq_first_pos, 2 * self.H, self.scale, ctx.status, window,
                                          keep_first=self.keep_first, out_float=maps)
            ops.diff_combine(attn, maps, self.H, self.lam, self.eps, out_scale)
        elif (not ctx.all_decode and N >= 4 * ctx.num_seqs
                and ops.attention_diff_tile_supports(self.H, self.G, self.dim, self.dv, ctx.dtype)):
            # prompt portions: a tile of a request's consecutive tokens per block shares the keys it reads
            ops.attention_diff_tile(attn, q, k_pool, v_pool, table, ctx.seq_starts, ctx.seq_rows, ctx.seq_first_pos,
                                    self.H, self.scale, self.lam, self.eps, out_scale, window, self.keep_first)
        else:
            NP, part_o, part_ml = self.partitions(ctx, N, cache.manager.max_len), None, None
            if NP > 1:
                part_o = ctx.buffers.take_flat("attn_part_o", N * self.H * 2 * NP * self.dv, torch.float32)
                part_ml = ctx.buffers.take_flat("attn_part_ml", N * self.H * 4 * NP, torch.float32)
            ops.attention_diff(attn, q, k_pool, v_pool, table, ctx.token_rows, ctx.positions, self.H, self.scale,
                               self.lam, self.eps, out_scale, window, self.keep_first, num_partitions=NP,
                               part_o=part_o, part_ml=part_ml)
        return Branch(self.o(ctx, attn, "branch", out="partial"))


register_part("mixer", "differential_attention", DifferentialAttention)
