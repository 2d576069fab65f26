"""Tiny Magedra configurations for the tests and their random weights.

The configurations differ from one another in every size and option: 1, 2, 3 and 8 residual streams and none
at all, branch factors above, below and equal to one, a logit scale and none; attention with 1, 2 and 4 query
heads per key/value head, key rows of 6 to 64 dims (multiples of the 16-byte vector and not), values smaller
and larger than a key row and beyond 128 dims, full, partial and no rotation; linear attention with key rows
that need 4, 8 and 16 state rows a thread; latents smaller and larger than 128 dims, and cached rows of exactly 64 and
128 dims (which the bfloat16 engine serves on the tensor cores); recurrences narrower and
wider than a block of 128 channels; layers with and without a feed-forward; layers that run an earlier
layer's weights (next to it and further on); and one model whose sizes are no multiple of 8.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch


def _gru(width):
    return {"width": width}


def _par(heads, kv, dim, vdim, scale, rh, rdim, rvdim, rot=None, base=None, ls=1.0, rs=1.0):
    left = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        left["rot"] = {"dims": rot, "base": base}
    return {"left": left, "right": {"heads": rh, "dim": rdim, "vdim": rvdim}, "left_scale": ls, "right_scale": rs}


def _lat(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
            "scale": scale, "rot": {"base": base, "dims": rot_dim}}


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _layer(kind, mixer, mlp, weights_of=None):
    l = {"type": kind, "mixer": mixer, "mlp": mlp}
    if weights_of is not None:
        l["weights_of"] = weights_of
    return l


_G0, _P0, _L0 = _gru(24), _par(4, 2, 16, 8, 0.3, 2, 12, 20, rot=8, base=100.0, ls=1.3, rs=0.8), _lat(3, 8, 4, 12, 16, 20, 0.35, 1000.0)
_P2 = _par(2, 1, 64, 32, 0.12, 3, 130, 8, rot=64, base=50000.0, ls=0.7, rs=1.1)
_L2 = _lat(4, 16, 8, 16, 24, 56, 0.2, 20000.0)      # a cached row of 8 + 56 = 64 dims

TINY = {
    # three streams; every mixer; layers run again next to their owner and later; a layer without a feed-forward
    "A": {"architecture": "Magedra", "vocab": 97, "width": 40, "norm": {"eps": 1e-6}, "residual_mult": 0.6,
          "streams": 3, "logit_scale": 1.5,
          "layers": [_layer("mingru", _G0, _dense(48, 1.5)), _layer("parallel", _P0, _dense(48, 1.5)),
                     _layer("parallel", _P0, _dense(48, 1.5), 1), _layer("latent_attention", _L0, None),
                     _layer("mingru", _G0, _dense(48, 1.5), 0), _layer("latent_attention", _L0, None, 3)]},
    # one stream (with reading, writing and mixing weights all the same), no logit scale, a branch factor of one;
    # one query head per key/value head, values of 130 dims, no rotation; a latent of 136 dims; a recurrence of
    # 130 channels; a linear attention head of 70 key dims
    "B": {"architecture": "Magedra", "vocab": 67, "width": 48, "norm": {"eps": 1e-5}, "residual_mult": 1.0, "streams": 1,
          "layers": [_layer("parallel", _par(6, 6, 8, 130, 0.4, 1, 70, 9), _dense(24, 0.7)),
                     _layer("latent_attention", _lat(2, 24, 6, 40, 12, 136, 0.15, 300.0), _dense(24, 0.7)),
                     _layer("mingru", _gru(130), None)]},
    # no streams at all: one residual; two query heads a group, key rows of 64 dims that all rotate; linear
    # attention with 130 key dims
    "C": {"architecture": "Magedra", "vocab": 300, "width": 64, "norm": {"eps": 1e-5}, "residual_mult": 0.5,
          "logit_scale": 0.25,
          "layers": [_layer("parallel", _P2, _dense(72, 1.2)), _layer("latent_attention", _L2, _dense(40, 1.2)),
                     _layer("parallel", _P2, _dense(72, 1.2), 0), _layer("mingru", _gru(64), _dense(72, 1.2))]},
    # a width, feed-forwards, heads, latents and a vocabulary that are no multiple of 8; two streams
    "D": {"architecture": "Magedra", "vocab": 53, "width": 36, "norm": {"eps": 1e-6}, "residual_mult": 1.2, "streams": 2,
          "logit_scale": 3.0,
          "layers": [_layer("latent_attention", _lat(2, 6, 2, 5, 10, 7, 0.4, 50.0), _dense(20, 1.0)),
                     _layer("parallel", _par(3, 3, 6, 10, 0.5, 2, 5, 7, rot=4, base=30.0, ls=0.9, rs=1.4), _dense(20, 1.0)),
                     _layer("mingru", _gru(11), _dense(20, 1.0)),
                     _layer("latent_attention", _lat(2, 6, 2, 5, 10, 7, 0.4, 50.0), _dense(20, 1.0), 0)]},
    # eight streams; four query heads a group; a talking matrix over eight heads
    "E": {"architecture": "Magedra", "vocab": 80, "width": 56, "norm": {"eps": 1e-6}, "residual_mult": 0.4, "streams": 8,
          "logit_scale": 2.0,
          "layers": [_layer("parallel", _par(8, 2, 32, 64, 0.18, 2, 32, 16, rot=16, base=1000.0, ls=1.0, rs=1.0), _dense(64, 2.5)),
                     _layer("mingru", _gru(40), _dense(64, 2.5)),
                     _layer("latent_attention", _lat(8, 32, 32, 64, 48, 96, 0.12, 5000.0), _dense(64, 2.5))]},   # a row of 128
}


def make_weights(cfg: dict, seed: int):
    """Random tensors for a configuration, scaled so that every mechanism matters: projections large enough for
    attention to be peaked and for the clamps to bite, biases of the size of the projections, gates and lower
    bounds spread over their range."""
    from socrates_b200.config import config_from_dict
    from socrates_b200.engine.model import Model
    from socrates_b200.weights.random_init import random_tensors
    params = Model(config_from_dict(cfg).plan()).parameters()
    w = random_tensors(params, seed)
    g = torch.Generator().manual_seed(seed + 1)
    for name in list(w):
        t = w[name].float()
        if name in ("embed", "head"):
            t = t * 20.0
        elif name.endswith(".b"):
            t = 0.5 * torch.randn(t.shape, generator=g)
        elif name.endswith(".talk"):
            t = torch.eye(t.shape[0]) * 0.8 + 0.4 * torch.randn(t.shape, generator=g)
        elif params[name].role == "matrix":
            t = t * 4.0
        # everything is stored as bfloat16, so both engines and the plain statement read equal values
        w[name] = t.to(torch.bfloat16)
    return w


def make_folder(tmp_path, name: str, seed: int = 5, cfg: dict = None):
    """(folder, config dict, weights as float64) of the tiny model `name`."""
    cfg = TINY[name] if cfg is None else cfg
    w = make_weights(cfg, seed)
    folder = Path(tmp_path) / f"magedra_{name}"
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_weights(folder, w)
    return folder, cfg, {k: v.double() for k, v in w.items()}


def save_weights(folder, w):
    from safetensors.torch import save_file
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in w.items()}, str(Path(folder) / "model.safetensors"))
