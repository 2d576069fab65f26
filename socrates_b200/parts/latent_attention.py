"""Attention through low-rank latents: what is cached per token is one latent vector and one rotated key
part, shared by all heads.

    c_q = rmsnorm(W_dq x) * w_dq ;  q = W_uq c_q            per head [key_dim that do not turn | rot_dim that turn]
    W_dkv x = [kv_rank | rot_dim] ;  c = rmsnorm(first part) * w_dkv ;  k_rot = rotate(last part)     (one per token)
    per head: k_h = W_uk,h c ,  v_h = W_uv,h c
    s_h(i, j) = (q_h(i)[:key_dim] . k_h(j) + rotate(q_h(i)[key_dim:]) . k_rot(j)) * scale ,  j <= i ,  softmax
    out = W_o concat_h(sum_j p_h(i, j) v_h(j))

Keys and values are never made: q_h . (W_uk,h c) = (W_uk,h^T q_h) . c, so the query is carried into the
latent space (a matrix per head), the cache holds the row [k_rot | c] as the ONE key head of `rot_dim +
kv_rank` dims with c again as its value, the engine's paged attention runs `heads` query heads over that one
head, and its output (sum_j p c_j per head) goes through W_uv,h afterwards.  The rows of W_uq are reordered
when the weights are bound so that every head's turning part comes first.  One kernel norms the latent, turns
the key part and the queries and writes the token's row into its pages.
Norms, angles, scores, weights and sums are float32; the per-head matrices accumulate in float32.  One exception, in
the bfloat16 engine only: prompt portions of layers whose cached row has 64 or 128 dims run on the tensor-core tile
kernel (the key rows serve as values too), where each softmax weight enters the value product as two bfloat16 terms.
Tensors: `<name>dq`, `dq.norm`, `uq`, `dkv`, `dkv.norm`, `uk`, `uv`, `o`.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..cache.manager import CacheNeeds, PagedKVSpec
from ..kernels import ops
from .base import Branch, ParamSpec, Part, build_part, register_part
from .linear import Linear


class LatentAttention(Part):
    out_buffer = "branch"

    def __init__(self, spec, name):
        super().__init__(spec, name)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.H, self.dn, self.dr, self.dv = int(p["num_heads"]), int(p["key_dim"]), int(p["rot_dim"]), int(p["value_dim"])
        self.q_rank, self.kv_rank = int(p["q_rank"]), int(p["kv_rank"])
        self.scale, self.eps = float(p["scale"]), float(p["norm_eps"])
        self.window: Optional[int] = p.get("window")
        self.position = build_part("position", p["position"], "")
        self.D = self.dr + self.kv_rank                  # the cached key row: [k_rot | c]
        if self.dr % 2:
            raise ValueError(f"{self.dr} turning dims are not even")
        if not (1 <= self.D <= 576 and self.kv_rank <= 256):
            raise ValueError(f"a cached row of {self.dr} + {self.kv_rank} dims; the kernels take up to 576, with a "
                             f"latent of up to 256")
        self.down: Optional[Linear] = None
        self.uq: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.uk = self.uv = self.q_gain = self.kv_gain = None

    def parameters(self) -> Dict[str, ParamSpec]:
        n, H = self.name, self.H
        return {
            n + "dq": ParamSpec((self.q_rank, self.hidden)), n + "dq.norm": ParamSpec((self.q_rank,), role="gain", init="gain"),
            n + "uq": ParamSpec((H * (self.dn + self.dr), self.q_rank)),
            n + "dkv": ParamSpec((self.kv_rank + self.dr, self.hidden)),
            n + "dkv.norm": ParamSpec((self.kv_rank,), role="gain", init="gain"),
            n + "uk": ParamSpec((H * self.dn, self.kv_rank)), n + "uv": ParamSpec((H * self.dv, self.kv_rank)),
            n + "o": ParamSpec((self.hidden, H * self.dv)),
        }

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        n, H, dn, dr = self.name, self.H, self.dn, self.dr
        self.down = Linear(torch.cat([tensors[n + "dq"], tensors[n + "dkv"]], dim=0))
        uq = tensors[n + "uq"].view(H, dn + dr, self.q_rank)
        self.uq = Linear(torch.cat([uq[:, dn:], uq[:, :dn]], dim=1).reshape(H * (dn + dr), self.q_rank).contiguous())
        self.uk, self.uv = tensors[n + "uk"].contiguous(), tensors[n + "uv"].contiguous()
        self.o = Linear(tensors[n + "o"])
        self.q_gain, self.kv_gain = tensors[n + "dq.norm"], tensors[n + "dkv.norm"]
        self.position.tables(self.o.weight.device)

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(paged=PagedKVSpec(1, self.D, self.window, self.kv_rank))

    def streamed_weights(self):
        return [self.down.weight, self.uq.weight, self.o.weight]

    def partitions(self, ctx, N: int, max_len: int) -> int:
        span = min(self.window or max_len, max_len)
        return max(1, min(16, (4 * ctx.num_sms) // max(1, N), -(-span // 64)))

    def forward(self, ctx, x: torch.Tensor, cache) -> Branch:
        N, H, D, rank, dr, dn = x.shape[0], self.H, self.D, self.kv_rank, self.dr, self.dn
        down = self.down(ctx, x, "la_down")                                  # [c_q raw | c raw | k_rot raw]
        cq = ctx.buffers.take("la_cq", N, (self.q_rank,), ctx.dtype)
        ops.segment_norm(down, [(0, self.q_rank, self.q_gain, [(cq, 0)])], self.eps)
        qf = self.uq(ctx, cq, "la_q")                                        # per head [turning | not turning]
        # the query heads as the attention kernel reads them: [q_rot | q carried into the latent space]
        q = ctx.buffers.take("la_qr", N, (H * D,), ctx.dtype)
        ops.head_matmul(q, dr, D, qf, dr, dn + dr, self.uk, H, transposed=True, carry=dr)
        k_pool, v_pool = cache.pools()
        table = cache.block_table()
        inv_freq, rotary_dim = self.position.tables(x.device)
        ops.latent_write(down, self.q_rank, self.q_rank + rank, rank, rotary_dim, self.kv_gain, self.eps, q, H,
                         inv_freq, self.position.neighbours, getattr(self.position, "magnitude", 1.0),
                         ctx.positions, ctx.token_rows, table, k_pool, v_pool)
        src, first, step = None, 0, rank                   # where the attention output lies: matrix, first column, head stride
        if (not ctx.all_decode and ctx.dtype == torch.bfloat16 and ctx.status is not None and D in (64, 128)
                and ops.attention_tcgen05_supports(H, 1, D, k_pool.shape[2])):
            # prompt portions in the bfloat16 engine whose cached row has 64 or 128 dims: the tensor-core tile kernel,
            # with the key rows [k_rot | c] as the values too, so that keys and values have one size; the head's
            # output is then sum_j p [k_rot | c]_j, of which only the latent part is carried on.  Scores are float32
            # sums over the bfloat16 q and k, softmax is float32, each weight enters the value product as two
            # bfloat16 terms.
            src = ctx.buffers.take("la_wide", N, (H * D,), ctx.dtype)
            ops.attention_prefill_tcgen05(src, q, k_pool, k_pool, table, ctx.seq_starts, ctx.seq_rows, ctx.seq_first_pos,
                                          H, self.scale, ctx.status, self.window or 0)
            first, step = dr, D
        elif (not ctx.all_decode and N >= 4 * ctx.num_seqs
                and ops.attention_bias_tile_supports(H, 1, D, rank, ctx.dtype)):
            src = ctx.buffers.take("la_lat", N, (H * rank,), ctx.dtype)
            ops.attention_bias_tile(src, q, k_pool, v_pool, table, ctx.seq_starts, ctx.seq_rows, ctx.seq_first_pos,
                                    H, self.scale, self.window or 0)
        else:
            src = ctx.buffers.take("la_lat", N, (H * rank,), ctx.dtype)
            NP, part_o, part_ml = self.partitions(ctx, N, cache.manager.max_len), None, None
            if NP > 1:
                part_o = ctx.buffers.take_flat("attn_part_o", N * H * NP * rank, torch.float32)
                part_ml = ctx.buffers.take_flat("attn_part_ml", N * H * NP * 2, torch.float32)
            ops.attention_bias(src, q, k_pool, v_pool, table, ctx.token_rows, ctx.positions, H, self.scale,
                               self.window or 0, num_partitions=NP, part_o=part_o, part_ml=part_ml)
        heads = ctx.buffers.take("la_heads", N, (H * self.dv,), ctx.dtype)
        ops.head_matmul(heads, 0, self.dv, src, first, step, self.uv, H, transposed=False)
        return Branch(self.o(ctx, heads, self.out_buffer, out="partial"))


register_part("mixer", "latent_attention", LatentAttention)
