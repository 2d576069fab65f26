"""A plain float64 statement of the Samerax decoder, one function per mechanism.

It shares nothing with the engine: weights are a mapping name -> tensor, a configuration is the
plain dictionary of config.json, a sequence is processed whole, and every attention weight is a
dense [T, T] matrix.  Slow and obvious on purpose.

    x_0   = embed[token] * embedding.scale
    layer:  x <- x + mixer(norm1(x)) ;  x <- x + ff(norm2(x))        (ff may be absent)
    mixer:  differential attention: two score maps per head over one set of values,
            o = softmax(S1) V - lambda * softmax(S2) V, normed per head, times (1 - diff)
    logits = cap * tanh(head(norm(x)) / cap)
"""

from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional

import torch

F64 = torch.float64


def rms_norm(x: torch.Tensor, gain: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if gain is None else y * gain


def yarn_frequencies(rot: Mapping) -> tuple:
    """Frequencies f_i, i < dims/2, and the factor on cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def dim_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    f = f / factor * ramp + f * (1.0 - ramp)
    return f, 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: Optional[Mapping]) -> torch.Tensor:
    """x [T, heads, dim]: the first rot.dims dims rotate, dim i with dim i + dims/2."""
    if not rot or int(rot["dims"]) == 0:
        return x
    dims = int(rot["dims"])
    f, mag = yarn_frequencies(rot)
    ang = positions.to(F64)[:, None] * f[None, :]                 # [T, dims/2]
    c, s = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    u, v = x[..., : dims // 2], x[..., dims // 2: dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def visible(T: int, size: Optional[int], keep_first: int) -> torch.Tensor:
    """[T, T] bool: query i (row) sees key j (column)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if size is not None:
        ok &= (i - j < size) | (j < keep_first)
    return ok


def softmax_map(q: torch.Tensor, k: torch.Tensor, scale: float, mask: torch.Tensor) -> torch.Tensor:
    """q [T, dim], k [T, dim] -> weights [T, T]."""
    s = (q @ k.T) * scale
    s = s.masked_fill(~mask, float("-inf"))
    return torch.softmax(s, dim=-1)


def diff_lambda(w: Mapping[str, torch.Tensor], pre: str, diff: float) -> float:
    d = lambda n: w[pre + n].to(F64)
    return float(torch.exp((d("lq1") * d("lk1")).sum()) - torch.exp((d("lq2") * d("lk2")).sum()) + diff)


def differential_heads(q, k, v, mask, scale: float, lam: float, diff: float, eps: float) -> torch.Tensor:
    """q [T, H, 2, dim], k [T, G, 2, dim], v [T, G, vdim], mask [T, T] -> [T, H, vdim]: per head the difference of
    two softmax maps over the same values, normed over the head's values, times (1 - diff)."""
    H, G = q.shape[1], k.shape[1]
    heads = []
    for hd in range(H):
        g = hd // (H // G)
        a1 = softmax_map(q[:, hd, 0], k[:, g, 0], scale, mask) @ v[:, g]
        a2 = softmax_map(q[:, hd, 1], k[:, g, 1], scale, mask) @ v[:, g]
        heads.append(rms_norm(a1 - lam * a2, None, eps) * (1.0 - diff))
    return torch.stack(heads, dim=1)


def attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], pre: str, m: Mapping, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, dim, vdim = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    lin = lambda n: h @ w[pre + n].to(F64).T + w[pre + n + ".b"].to(F64)
    pos = torch.arange(T)
    rot = m.get("rot")
    q = rotate(lin("q").view(T, H * 2, dim), pos, rot).view(T, H, 2, dim)
    k = rotate(lin("k").view(T, G * 2, dim), pos, rot).view(T, G, 2, dim)
    v = lin("v").view(T, G, vdim)
    mask_cfg = m.get("mask") or {}
    mask = visible(T, mask_cfg.get("size"), int(mask_cfg.get("keep_first", 0)))
    diff = float(m["diff"])
    o = differential_heads(q, k, v, mask, float(m["scale"]), diff_lambda(w, pre, diff), diff, eps)
    return o.reshape(T, H * vdim) @ w[pre + "o"].to(F64).T


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def gated_ff(h: torch.Tensor, w: Mapping[str, torch.Tensor], pre: str) -> torch.Tensor:
    d = lambda n: w[pre + n].to(F64)
    return (silu(h @ d("gate").T) * (h @ d("up").T)) @ d("down").T


def table_experts(h: torch.Tensor, tokens: torch.Tensor, w: Mapping[str, torch.Tensor], pre: str,
                  top: int) -> torch.Tensor:
    """Every token id names its experts in a table; each counts 1/top."""
    table = w[pre + "table"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in table[int(tokens[t])].tolist():
            out[t] += gated_ff(h[t:t + 1], w, f"{pre}e{int(e)}.")[0] / top
    return out


def feed_forward(h, tokens, w, pre, mlp) -> torch.Tensor:
    if mlp["kind"] == "dense":
        return gated_ff(h, w, pre)
    return table_experts(h, tokens, w, pre, int(mlp["router"]["top"]))


def forward(cfg: Mapping, w: Mapping[str, torch.Tensor], tokens, return_layers: bool = False):
    """Logits [T, vocab] (float64) of one sequence; with `return_layers` also the stream after every layer run."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = float(cfg["norm"]["eps"])
    x = w["embed"].to(F64)[tokens] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    streams: List[torch.Tensor] = []
    for i, layer in enumerate(cfg["layers"]):
        src = layer.get("weights_of")
        pre = f"l{i if src is None else int(src)}."
        if layer["type"] != "attention":
            raise ValueError(layer["type"])
        x = x + attention(rms_norm(x, w[pre + "norm1"].to(F64), eps), w, pre + "mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            x = x + feed_forward(rms_norm(x, w[pre + "norm2"].to(F64), eps), tokens, w, pre + "mlp.", layer["mlp"])
        streams.append(x.clone())
    z = rms_norm(x, w["final.norm"].to(F64), eps) @ w["head"].to(F64).T
    cap = cfg.get("logit_softcap")
    if cap:
        z = float(cap) * torch.tanh(z / float(cap))
    return (z, torch.stack(streams)) if return_layers else z
