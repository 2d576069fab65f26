"""Typed configuration of the Magedra decoder, read from its config.json.

The file names the design under "architecture" and gives `vocab`, `width`, `norm.eps`, `residual_mult`,
`streams`, `logit_scale` and a list `layers`; each entry has a `type` ("mingru", "parallel" or
"latent_attention"), the mixer's sizes under `mixer` and its feed-forward under `mlp` (null: none; `kind`
"dense" with `ff` and `limit`).  An entry with `weights_of: j` has no tensors of its own: it runs layer j's
weights with a cache and state of its own.  Mixers give:

  * mingru: `width`;
  * parallel: `left` (`heads`, `kv_heads`, `dim`, `vdim`, `scale`, optionally `rot`: `dims`, `base`),
    `right` (`heads`, `dim`, `vdim`), `left_scale`, `right_scale`;
  * latent_attention: `heads`, `dim`, `rot_dim`, `vdim`, `q_rank`, `kv_rank`, `scale`, `rot.base`.

Every size and every constant a checkpoint can vary comes from there; what the design fixes is written in
`plan()`:

  * the looked-up embedding rows pass a layer norm (tensor `embed.norm`) before they become the residual;
  * every norm in front of a sublayer, after the embedding and in front of the head is a layer norm with a
    gain and no bias;
  * the residual is `streams` streams with learned reading, writing and mixing weights per sublayer
    (arrangement "hyper_connections"; without `streams` one residual), every branch times `residual_mult`;
  * "mingru" is the mixer "min_gru" with biases on the gate and the candidate;
  * "parallel" is "scaled_sum" of a "talking_attention" (rotation in halves of the first `rot.dims` dims,
    scores mixed across heads, a sigmoid gate on the heads, no window) under `left.` and a
    "gated_linear_attention" under `right.`;
  * "latent_attention": rotation in neighbouring pairs of the `rot_dim` turning dims, RMS norms on both latents;
  * feed-forwards are "clamped_glu" with alpha 1.702 and the value shifted by one;
  * the logits are multiplied by `logit_scale`.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Dict, Mapping, Optional, Tuple

from .bofusun import _freeze, _need
from .plan import LayerSpec, ModelPlan, PartSpec, RunEntry
from .qwen3 import ConfigError

MIXERS = ("mingru", "parallel", "latent_attention")


@dataclass(frozen=True)
class MagedraLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]
    weights_of: Optional[int] = None

    def __hash__(self):
        return hash((self.type, _freeze(self.mixer), _freeze(self.mlp), self.weights_of))


@dataclass(frozen=True)
class MagedraConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    streams: int                     # 0: one residual
    logit_scale: float
    layers: Tuple[MagedraLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()

    architecture = "Magedra"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "MagedraConfig":
        _need(d, ("vocab", "width", "norm", "layers"), "config.json")
        _need(d["norm"], ("eps",), "config.json norm")
        layers = []
        for i, l in enumerate(d["layers"]):
            _need(l, ("type", "mixer"), f"layers[{i}]")
            src = l.get("weights_of")
            layers.append(MagedraLayer(str(l["type"]), dict(l["mixer"]),
                                       dict(l["mlp"]) if l.get("mlp") is not None else None,
                                       None if src is None else int(src)))
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        cfg = cls(vocab=int(d["vocab"]), width=int(d["width"]), norm_eps=float(d["norm"]["eps"]),
                  residual_mult=float(d.get("residual_mult", 1.0)), streams=int(d.get("streams") or 0),
                  logit_scale=float(d.get("logit_scale", 1.0)), layers=tuple(layers), eos_token_ids=eos_ids)
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path) -> "MagedraConfig":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        return cls.from_dict(json.loads(path.read_text()))

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ConfigError("vocab, width and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        if not 0 <= self.streams <= 8:
            raise ConfigError(f"streams={self.streams}: the engine folds up to 8 residual streams")
        for i, l in enumerate(self.layers):
            m, where = l.mixer, f"layers[{i}].mixer"
            if l.type not in MIXERS:
                raise ConfigError(f"layers[{i}].type={l.type!r} is not a known mixer; known: {', '.join(MIXERS)}")
            if l.type == "mingru":
                _need(m, ("width",), where)
                if int(m["width"]) < 1:
                    raise ConfigError(f"{where}: width must be positive")
            elif l.type == "parallel":
                _need(m, ("left", "right", "left_scale", "right_scale"), where)
                a, b = m["left"], m["right"]
                _need(a, ("heads", "kv_heads", "dim", "vdim", "scale"), where + ".left")
                _need(b, ("heads", "dim", "vdim"), where + ".right")
                if int(a["heads"]) < 1 or int(a["kv_heads"]) < 1 or int(a["heads"]) % int(a["kv_heads"]):
                    raise ConfigError(f"{where}.left: heads is no multiple of kv_heads")
                rot = a.get("rot")
                if rot is not None:
                    _need(rot, ("dims", "base"), where + ".left.rot")
                    if int(rot["dims"]) % 2 or not 0 <= int(rot["dims"]) <= int(a["dim"]):
                        raise ConfigError(f"{where}.left: rot.dims must be even and at most dim")
            else:
                _need(m, ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale"), where)
                if int(m["rot_dim"]) % 2:
                    raise ConfigError(f"{where}: rot_dim must be even")
                if int(m["rot_dim"]) > 0:
                    _need(m.get("rot") or {}, ("base",), where + ".rot")
                    dims = (m.get("rot") or {}).get("dims")
                    if dims is not None and int(dims) != int(m["rot_dim"]):
                        raise ConfigError(f"{where}: rot.dims={dims} differs from rot_dim={m['rot_dim']}")
            if l.mlp is not None:
                mw = f"layers[{i}].mlp"
                _need(l.mlp, ("kind",), mw)
                if l.mlp["kind"] != "dense":
                    raise ConfigError(f"{mw}.kind={l.mlp['kind']!r} is not supported; known: dense")
                _need(l.mlp, ("ff", "limit"), mw)
            if l.weights_of is not None:
                j = l.weights_of
                if not 0 <= j < i or self.layers[j].weights_of is not None:
                    raise ConfigError(f"layers[{i}].weights_of={j} does not name an earlier layer with tensors of its own")
                if (l.mlp is None) != (self.layers[j].mlp is None):
                    raise ConfigError(f"layers[{i}] runs the weights of layer {j}, whose feed-forward it lacks or adds")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        layers = []
        for l in self.layers:
            e: Dict[str, Any] = {"type": l.type, "mixer": json.loads(json.dumps(l.mixer)),
                                 "mlp": json.loads(json.dumps(l.mlp)) if l.mlp is not None else None}
            if l.weights_of is not None:
                e["weights_of"] = l.weights_of
            layers.append(e)
        d: Dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult, "logit_scale": self.logit_scale,
            "layers": layers,
        }
        if self.streams:
            d["streams"] = self.streams
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # --------------------------------------------------------------------- plan
    def _norm(self, name: str) -> PartSpec:
        return PartSpec("layernorm", {"dim": self.width, "eps": self.norm_eps, "suffix": ""}, name)

    def _mixer(self, l: MagedraLayer) -> PartSpec:
        m = l.mixer
        if l.type == "mingru":
            return PartSpec("min_gru", {"hidden_size": self.width, "width": int(m["width"]), "bias": True}, "mix.")
        if l.type == "parallel":
            a, b = m["left"], m["right"]
            rot = a.get("rot")
            if rot is not None and int(rot["dims"]) > 0:
                position = PartSpec("rotary", {"head_dim": int(a["dim"]), "rotary_dim": int(rot["dims"]),
                                               "theta": float(rot["base"]), "pairing": "halves",
                                               "table_precision": "float64"})
            else:
                position = PartSpec("none", {})
            left = PartSpec("talking_attention", {
                "hidden_size": self.width, "num_heads": int(a["heads"]), "num_kv_heads": int(a["kv_heads"]),
                "key_dim": int(a["dim"]), "value_dim": int(a["vdim"]), "scale": float(a["scale"]), "gate": True,
                "window": None, "position": position}, "left.")
            right = PartSpec("gated_linear_attention", {
                "hidden_size": self.width, "num_heads": int(b["heads"]), "key_dim": int(b["dim"]),
                "value_dim": int(b["vdim"]), "norm_eps": self.norm_eps}, "right.")
            return PartSpec("scaled_sum", {"hidden_size": self.width, "branches": (left, right),
                                           "scales": (float(m["left_scale"]), float(m["right_scale"]))}, "mix.")
        dr, rank = int(m["rot_dim"]), int(m["kv_rank"])
        if dr > 0:
            position = PartSpec("rotary", {"head_dim": dr + rank, "rotary_dim": dr, "theta": float(m["rot"]["base"]),
                                           "pairing": "neighbours", "table_precision": "float64"})
        else:
            position = PartSpec("none", {})
        return PartSpec("latent_attention", {
            "hidden_size": self.width, "num_heads": int(m["heads"]), "key_dim": int(m["dim"]), "rot_dim": dr,
            "value_dim": int(m["vdim"]), "q_rank": int(m["q_rank"]), "kv_rank": rank, "scale": float(m["scale"]),
            "norm_eps": self.norm_eps, "window": None, "position": position}, "mix.")

    def _feed_forward(self, l: MagedraLayer) -> Optional[PartSpec]:
        if l.mlp is None:
            return None
        return PartSpec("clamped_glu", {"hidden_size": self.width, "intermediate_size": int(l.mlp["ff"]),
                                        "limit": float(l.mlp["limit"]), "alpha": 1.702, "offset": 1.0}, "mlp.")

    def plan(self) -> ModelPlan:
        layers, order, index_of = [], [], {}
        arrangement = {"streams": self.streams, "residual_mult": self.residual_mult, "hidden_size": self.width}
        for i, l in enumerate(self.layers):
            j = l.weights_of
            if j is not None and (l.type, _freeze(l.mixer), _freeze(l.mlp)) == \
                    (self.layers[j].type, _freeze(self.layers[j].mixer), _freeze(self.layers[j].mlp)):
                order.append(RunEntry(index_of[j]))        # the same layer again, with a cache of its own
                continue
            # (an entry that names another layer's weights but other constants is a layer of its own
            # that reads the same tensors)
            ff = self._feed_forward(l)
            norms = (self._norm("norm1"),) if ff is None else (self._norm("norm1"), self._norm("norm2"))
            index_of[i] = len(layers)
            layers.append(LayerSpec("hyper_connections", f"l{i if j is None else j}.", norms, self._mixer(l), ff,
                                    params=arrangement))
            order.append(RunEntry(index_of[i]))
        plan = ModelPlan(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            embedding=PartSpec("normed_embedding", {"vocab_size": self.vocab, "hidden_size": self.width, "suffix": "",
                                                    "norm": self._norm(".norm")}, "embed"),
            layers=tuple(layers), order=tuple(order),
            final_norm=self._norm("final.norm"),
            head=PartSpec("lm_head", {"hidden_size": self.width, "vocab_size": self.vocab, "tied_to": None,
                                      "suffix": "", "scale": self.logit_scale}, "head"),
        )
        plan.validate()
        return plan

    def describe(self) -> dict:
        return self.to_dict()
