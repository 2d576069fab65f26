"""A plain float64 statement of the Magedra decoder, one function per mechanism.

It shares nothing with the engine: weights are a mapping name -> tensor, a configuration is the
plain dictionary of config.json, a sequence is processed whole, recurrences walk token by token
and every attention weight is a dense [T, T] matrix.  Slow and obvious on purpose.

    x_1 .. x_s = layer_norm(embed[token]) * w            (s residual streams, all equal at first)
    sublayer q of a layer (1: mixer, 2: feed-forward):
        u = sum_s in_q[s] x_s ;  y = sublayer(layer_norm(u))
        x_t <- sum_s mix_q[s, t] x_s + m * out_q[t] * y                 (all t at once)
    mixers: "mingru" (a gated recurrence per channel), "parallel" (softmax attention whose scores
            are mixed across heads, beside a gated linear attention), "latent_attention"
    logits = head(layer_norm(sum_s x_s)) * logit_scale
"""

from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional

import torch

F64 = torch.float64


def layer_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(mean of squared deviations + eps) * gain; no bias."""
    d = x - x.mean(-1, keepdim=True)
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * gain


def rms_norm(x: torch.Tensor, gain: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if gain is None else y * gain


def sigmoid(x):
    return 1.0 / (1.0 + torch.exp(-x))


def silu(x):
    return x * sigmoid(x)


def frequencies(rot: Mapping) -> torch.Tensor:
    dims = int(rot["dims"])
    return float(rot["base"]) ** (-2.0 * torch.arange(dims // 2, dtype=F64) / dims)


def rotate_halves(x: torch.Tensor, positions: torch.Tensor, rot: Optional[Mapping]) -> torch.Tensor:
    """x [T, heads, dim]: of the first rot.dims dims, dim i turns with dim i + dims/2; the rest pass."""
    if not rot or int(rot["dims"]) == 0:
        return x
    dims = int(rot["dims"])
    ang = positions.to(F64)[:, None] * frequencies(rot)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., : dims // 2], x[..., dims // 2: dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, rot: Optional[Mapping]) -> torch.Tensor:
    """x [T, heads, dim]: of the first rot.dims dims, dim 2i turns with dim 2i + 1; the rest pass."""
    if not rot or int(rot["dims"]) == 0:
        return x
    dims = int(rot["dims"])
    ang = positions.to(F64)[:, None] * frequencies(rot)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def causal_softmax(scores: torch.Tensor) -> torch.Tensor:
    """scores [heads, T, T] (query, key): key j is visible to query i when j <= i."""
    T = scores.shape[-1]
    seen = torch.ones(T, T, dtype=torch.bool).tril()
    return torch.softmax(scores.masked_fill(~seen, -math.inf), dim=-1)


# ------------------------------------------------------------------------------------------ mixers
def min_gru(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, state: Optional[torch.Tensor] = None):
    """z = sigmoid(W_z h + b_z); u = W_x h + b_x; candidate = u + 1/2 (u >= 0) or sigmoid(u) (u < 0);
    S_t = (1 - z) S_(t-1) + z candidate; out = W_o (S_t * silu(W_g h)).  Returns (out, last state)."""
    z = sigmoid(h @ w[p + "z"].T + w[p + "z.b"])
    u = h @ w[p + "x"].T + w[p + "x.b"]
    cand = torch.where(u >= 0, u + 0.5, sigmoid(u))
    gate = silu(h @ w[p + "g"].T)
    S = torch.zeros(z.shape[1], dtype=h.dtype) if state is None else state.clone()
    rows = []
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        rows.append(S * gate[t])
    return torch.stack(rows) @ w[p + "o"].T, S


def talking_attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping,
                      positions: torch.Tensor) -> torch.Tensor:
    """Grouped-query softmax attention whose scaled scores are mixed across heads before the mask and
    the softmax (score_h <- sum_g talk[h, g] score_g), with a sigmoid gate on the concatenated heads."""
    T = h.shape[0]
    H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = rotate_halves((h @ w[p + "q"].T).view(T, H, dk), positions, m.get("rot"))
    k = rotate_halves((h @ w[p + "k"].T).view(T, G, dk), positions, m.get("rot"))
    v = (h @ w[p + "v"].T).view(T, G, dv)
    kv_of = torch.arange(H) // (H // G)
    scores = torch.einsum("ihd,jhd->hij", q, k[:, kv_of]) * float(m["scale"])
    scores = torch.einsum("hg,gij->hij", w[p + "talk"], scores)
    o = torch.einsum("hij,jhe->ihe", causal_softmax(scores), v[:, kv_of]).reshape(T, H * dv)
    return (o * sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def gated_linear_attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping, eps: float,
                           state: Optional[torch.Tensor] = None):
    """q = silu(W_q h); v = W_v h; f = l + (1 - l) sigmoid(W_f h + b_f) per head and channel;
    S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T; o_t = S_t^T q_t; each head's o is RMS-normed over its
    value dims with one gain shared by the heads.  Returns (out, last state [heads, dim, vdim])."""
    T = h.shape[0]
    H, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(h @ w[p + "q"].T).view(T, H, dk)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    low = w[p + "lower"]
    f = (low + (1.0 - low) * sigmoid(h @ w[p + "f"].T + w[p + "f.b"])).view(T, H, dk)
    S = torch.zeros(H, dk, dv, dtype=h.dtype) if state is None else state.clone()
    rows = []
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        rows.append(torch.einsum("hde,hd->he", S, q[t]))
    o = rms_norm(torch.stack(rows), w[p + "norm"], eps).reshape(T, H * dv)
    return o @ w[p + "o"].T, S


def parallel_mixer(h, w, p, m, eps, positions):
    left = talking_attention(h, w, p + "left.", m["left"], positions)
    right, _ = gated_linear_attention(h, w, p + "right.", m["right"], eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def latent_attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping, eps: float,
                     positions: torch.Tensor) -> torch.Tensor:
    """Queries and keys/values through low-rank latents; every head's query and key have `dim` dims that
    do not turn and `rot_dim` dims that do (in neighbouring pairs); the turning key part is one vector
    shared by the heads.  Written without any absorption: keys and values are made from the latent."""
    T = h.shape[0]
    H, dn, dr, dv, rank = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    rot = {"dims": dr, "base": m["rot"]["base"]}
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).view(T, H, dn + dr)
    q_rot = rotate_pairs(q[..., dn:], positions, rot)
    down = h @ w[p + "dkv"].T
    c = rms_norm(down[:, :rank], w[p + "dkv.norm"], eps)
    k_rot = rotate_pairs(down[:, rank:].view(T, 1, dr), positions, rot)[:, 0]
    k = (c @ w[p + "uk"].T).view(T, H, dn)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q[..., :dn], k) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * float(m["scale"])
    o = torch.einsum("hij,jhe->ihe", causal_softmax(scores), v).reshape(T, H * dv)
    return o @ w[p + "o"].T


def feed_forward(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, mlp: Mapping) -> torch.Tensor:
    """g = min(W_g h + b, limit); u = clamp(W_u h + b, -limit, limit); down(g sigmoid(1.702 g) (u + 1)) + b."""
    lim = float(mlp["limit"])
    g = (h @ w[p + "gate"].T + w[p + "gate.b"]).clamp(max=lim)
    u = (h @ w[p + "up"].T + w[p + "up.b"]).clamp(-lim, lim)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T + w[p + "down.b"]


# ------------------------------------------------------------------------------------------ the model
def mixer(kind: str, h, w, p, m, eps, positions):
    if kind == "mingru":
        return min_gru(h, w, p)[0]
    if kind == "parallel":
        return parallel_mixer(h, w, p, m, eps, positions)
    if kind == "latent_attention":
        return latent_attention(h, w, p, m, eps, positions)
    raise ValueError(kind)


def hyper_step(xs: torch.Tensor, y_fn, w, p: str, mult: float) -> torch.Tensor:
    """xs [s, T, d]: read the streams with `in`, run the sublayer, mix the streams and write with `out`."""
    u = torch.einsum("s,std->td", w[p + "in"], xs)
    y = y_fn(u)
    return torch.einsum("st,snd->tnd", w[p + "mix"], xs) + mult * w[p + "out"][:, None, None] * y[None]


def forward(config: Mapping, weights: Mapping[str, torch.Tensor], tokens: List[int], dtype=F64,
            layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  `layers_out` collects the residual (the sum of the
    streams) after every layer run."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps, mult = float(config["norm"]["eps"]), float(config.get("residual_mult", 1.0))
    streams = config.get("streams")
    T = len(tokens)
    positions = torch.arange(T)
    x = layer_norm(w["embed"][torch.tensor(tokens)], w["embed.norm"], eps)
    xs = x[None].repeat(int(streams), 1, 1) if streams else None
    for i, l in enumerate(config["layers"]):
        src = l.get("weights_of")
        p = f"l{i if src is None else src}."

        def run_mixer(u, l=l, p=p):
            return mixer(l["type"], layer_norm(u, w[p + "norm1"], eps), w, p + "mix.", l["mixer"], eps, positions)

        def run_ff(u, l=l, p=p):
            return feed_forward(layer_norm(u, w[p + "norm2"], eps), w, p + "mlp.", l["mlp"])

        if streams:
            xs = hyper_step(xs, run_mixer, w, p + "hc1.", mult)
            if l.get("mlp") is not None:
                xs = hyper_step(xs, run_ff, w, p + "hc2.", mult)
            x = xs.sum(0)
        else:
            x = x + mult * run_mixer(x)
            if l.get("mlp") is not None:
                x = x + mult * run_ff(x)
        if layers_out is not None:
            layers_out.append(x.clone())
    return (layer_norm(x, w["final.norm"], eps) @ w["head"].T) * float(config.get("logit_scale", 1.0))
