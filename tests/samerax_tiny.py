"""Tiny Samerax configurations for the tests and their random weights.

The configurations differ from one another in every size and option: head counts and groups of 1, 2
and 3 query heads per key/value head, maps of 8 to 128 dims (multiples of the 16-byte vector and not),
value heads smaller than, equal to and larger than a key row (one beyond 128 dims; equal ones of 64 and 128 that the
bfloat16 engine serves on the tensor cores), full, partial
and no rotation, with and without stretched frequencies, windows shorter than a page, longer than a
chunk of 128 keys and absent, kept first keys of 0, 1, a whole page and more than the window, dense,
routed and no feed-forwards, top-1, top = every expert, layers that run an earlier layer's weights
(next to it and further on), logits with and without a cap, and one model whose sizes are no multiple of 8.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch


def _att(heads, kv, dim, vdim, scale, diff, rot=None, base=None, scaling=None, size=None, keep=0):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if rot is not None:
        m["rot"] = {"dims": rot, "base": base}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if size is not None:
        m["mask"] = {"size": size, "keep_first": keep}
    return m


def _moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _layer(mixer, mlp, weights_of=None):
    l = {"type": "attention", "mixer": mixer, "mlp": mlp}
    if weights_of is not None:
        l["weights_of"] = weights_of
    return l


_A0 = _att(6, 2, 8, 24, 0.4, 0.3, rot=6, base=100.0, scaling=(4.0, 32, 8.0, 1.0), size=37, keep=5)
_A1 = _att(2, 1, 16, 8, 0.3, 0.7, size=20, keep=0)
_C0 = _att(4, 2, 64, 32, 0.15, 0.45, rot=32, base=50000.0, scaling=(8.0, 64, 4.0, 0.5), size=130, keep=33)
_D0 = _att(2, 1, 64, 128, 0.1, 0.25, rot=64, base=1000.0, size=100, keep=65)
_D1 = _att(6, 3, 32, 64, 0.2, 0.4, rot=8, base=100.0, scaling=(2.0, 16, 4.0, 1.0), size=70, keep=9)

_E0 = _att(3, 1, 6, 10, 0.4, 0.35, rot=4, base=1000.0, scaling=(3.0, 24, 6.0, 1.0), size=21, keep=3)
_E1 = _att(2, 2, 10, 6, 0.3, 0.55, rot=10, base=300.0, size=50, keep=7)

TINY = {
    # three query heads a group, partial stretched rotation, a window with a few kept keys; layers run again
    # (next to their owner and later); a layer without a feed-forward; maps of 12 dims (no 16-byte rows in bfloat16)
    "A": {"architecture": "Samerax", "vocab": 101, "width": 48, "norm": {"eps": 1e-6}, "embedding": {"scale": 2.5},
          "logit_softcap": 20.0,
          "layers": [_layer(_A0, _dense(40)), _layer(_A1, _moe(16, 5, 2)), _layer(_A0, _dense(40), 0),
                     _layer(_A1, _moe(16, 5, 2), 1),
                     _layer(_att(3, 3, 12, 40, 0.35, 0.5, rot=12, base=10000.0), None),
                     _layer(_A0, _dense(40), 0)]},
    # no cap on the logits, no scale on the embedding, value heads of 130 dims, a window of exactly one page that
    # keeps a whole page, top-1 routing, routing to every expert, full rotation without stretching
    "B": {"architecture": "Samerax", "vocab": 67, "width": 40, "norm": {"eps": 1e-5},
          "layers": [_layer(_att(2, 2, 24, 130, 0.2, 0.6, rot=24, base=500.0, size=16, keep=16), _moe(8, 3, 1)),
                     _layer(_att(5, 1, 8, 16, 0.5, 0.2, size=9, keep=40), _moe(24, 2, 2)),
                     _layer(_att(2, 2, 24, 130, 0.2, 0.6, rot=24, base=500.0, size=16, keep=16), _moe(8, 3, 1), 0)]},
    # maps of 64 dims, two heads a group, a window longer than a chunk of keys with 33 kept keys
    "C": {"architecture": "Samerax", "vocab": 300, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.5},
          "logit_softcap": 8.0,
          "layers": [_layer(_C0, _moe(32, 4, 3)), _layer(_C0, _moe(32, 4, 3), 0), _layer(_C0, _dense(72))]},
    # key rows and value heads of one size, 128 and 64: in the bfloat16 engine prompt portions of these layers run on
    # the tensor-core attention kernel; kept keys that fill a key tile of 64 and one more, and a few only
    "D": {"architecture": "Samerax", "vocab": 80, "width": 96, "norm": {"eps": 1e-6}, "embedding": {"scale": 4.0},
          "logit_softcap": 50.0, "layers": [_layer(_D0, _dense(64)), _layer(_D1, _moe(24, 3, 2)), _layer(_D0, _dense(64), 0)]},
    # a width, feed-forwards, maps and values that are no multiple of 8 (no 16-byte rows anywhere in bfloat16), an odd
    # vocabulary, three of seven experts
    "E": {"architecture": "Samerax", "vocab": 53, "width": 36, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.5},
          "logit_softcap": 12.0, "layers": [_layer(_E0, _dense(20)), _layer(_E1, _moe(12, 7, 3)), _layer(_E0, _dense(20), 0)]},
}


def make_weights(cfg: dict, seed: int):
    """Random tensors for a configuration, scaled so that every mechanism matters: projections large enough
    for attention to be peaked, biases of the size of the projections, lambda terms of order one."""
    from socrates_b200.config import config_from_dict
    from socrates_b200.engine.model import Model
    from socrates_b200.weights.random_init import random_tensors
    params = Model(config_from_dict(cfg).plan()).parameters()
    w = random_tensors(params, seed)
    g = torch.Generator().manual_seed(seed + 1)
    for name in list(w):
        t = w[name]
        if params[name].role == "int":
            continue
        t = t.float()
        if name == "embed":
            t = t * 20.0
        elif name == "head":
            t = t * 20.0                       # logits large enough for the cap to bend them
        elif name.endswith(".b"):
            t = 0.5 * torch.randn(t.shape, generator=g)
        elif name.endswith((".lq1", ".lk1", ".lq2", ".lk2")):
            t = 0.4 * torch.randn(t.shape, generator=g)
        elif params[name].role == "matrix":
            t = t * 4.0
        # everything is stored as bfloat16, so both engines and the plain statement read equal values
        w[name] = t.to(torch.bfloat16)
    return w


def make_folder(tmp_path, name: str, seed: int = 5, cfg: dict = None):
    """(folder, config dict, weights as float64; tables stay integers) of the tiny model `name`."""
    cfg = TINY[name] if cfg is None else cfg
    w = make_weights(cfg, seed)
    folder = Path(tmp_path) / f"samerax_{name}"
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_weights(folder, w)
    return folder, cfg, {k: (v if v.dtype == torch.int32 else v.double()) for k, v in w.items()}


def save_weights(folder, w):
    from safetensors.torch import save_file
    save_file({k: (v if v.dtype == torch.int32 else v.to(torch.bfloat16)).contiguous() for k, v in w.items()},
              str(Path(folder) / "model.safetensors"))
