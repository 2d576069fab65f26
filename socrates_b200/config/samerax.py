"""Typed configuration of the Samerax decoder, read from its config.json.

The file names the design under "architecture" and gives `vocab`, `width`, `norm.eps`,
`embedding.scale`, `logit_softcap` and a list `layers`; each entry has a `type` ("attention"), the
mixer's sizes under `mixer` and its feed-forward under `mlp` (null: none; `kind` "dense" with `ff`,
or "moe" with `expert.ff` and `router`: `experts`, `top`).  An entry with `weights_of: j` has no
tensors of its own: it runs layer j's weights with a cache of its own.  A mixer gives `heads`,
`kv_heads`, `dim` (of one score map), `vdim`, `scale`, `diff`, optionally `rot` (`dims`, `base`,
optionally `scaling`: `factor`, `original`, `fast`, `slow`) and `mask` (`size`, `keep_first`).
Every size and every constant a checkpoint can vary comes from there; what the design fixes is
written in `plan()`:

  * the looked-up embedding rows are multiplied by `embedding.scale`;
  * a layer is x + mixer(norm1(x)), then x + ff(norm2(x)): RMS norms with plain gains in front of
    the branches (arrangement "pre_norm"; "pre_norm_mixer" for a layer without a feed-forward);
  * attention ("differential_attention"): two score maps per head over one set of values, biases on
    q, k and v, rotation in halves of the first `rot.dims` dims of every map with stretched
    frequencies, a sliding window that also keeps the first keys, the head norm's eps = norm.eps;
  * feed-forwards are gated with SiLU; the routed one ("routed_experts") takes every token's experts
    from a table by token id, each weighing 1 / top;
  * the logits are capped: c * tanh(logits / c).
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Dict, Mapping, Optional, Tuple

from .bofusun import _freeze, _need
from .plan import LayerSpec, ModelPlan, PartSpec, RunEntry
from .qwen3 import ConfigError


@dataclass(frozen=True)
class SameraxLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]
    weights_of: Optional[int] = None

    def __hash__(self):
        return hash((self.type, _freeze(self.mixer), _freeze(self.mlp), self.weights_of))


@dataclass(frozen=True)
class SameraxConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_softcap: Optional[float]
    layers: Tuple[SameraxLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()

    architecture = "Samerax"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "SameraxConfig":
        _need(d, ("vocab", "width", "norm", "layers"), "config.json")
        _need(d["norm"], ("eps",), "config.json norm")
        layers = []
        for i, l in enumerate(d["layers"]):
            _need(l, ("type", "mixer"), f"layers[{i}]")
            src = l.get("weights_of")
            layers.append(SameraxLayer(str(l["type"]), dict(l["mixer"]),
                                       dict(l["mlp"]) if l.get("mlp") is not None else None,
                                       None if src is None else int(src)))
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        cap = d.get("logit_softcap")
        cfg = cls(vocab=int(d["vocab"]), width=int(d["width"]), norm_eps=float(d["norm"]["eps"]),
                  embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)),
                  logit_softcap=float(cap) if cap else None, layers=tuple(layers), eos_token_ids=eos_ids)
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path) -> "SameraxConfig":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        return cls.from_dict(json.loads(path.read_text()))

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ConfigError("vocab, width and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        if self.logit_softcap is not None and not self.logit_softcap > 0:
            raise ConfigError("logit_softcap must be positive")
        for i, l in enumerate(self.layers):
            m, where = l.mixer, f"layers[{i}].mixer"
            if l.type != "attention":
                raise ConfigError(f"layers[{i}].type={l.type!r} is not a known mixer; known: attention")
            _need(m, ("heads", "kv_heads", "dim", "vdim", "scale", "diff"), where)
            if int(m["heads"]) < 1 or int(m["kv_heads"]) < 1 or int(m["heads"]) % int(m["kv_heads"]):
                raise ConfigError(f"{where}: heads is no multiple of kv_heads")
            rot = m.get("rot")
            if rot is not None:
                _need(rot, ("dims", "base"), where + ".rot")
                if int(rot["dims"]) % 2 or not 0 <= int(rot["dims"]) <= int(m["dim"]):
                    raise ConfigError(f"{where}: rot.dims must be even and at most dim")
                if rot.get("scaling"):
                    _need(rot["scaling"], ("factor", "original", "fast", "slow"), where + ".rot.scaling")
            mask = m.get("mask")
            if mask is not None:
                _need(mask, ("size",), where + ".mask")
                if int(mask["size"]) < 1 or int(mask.get("keep_first", 0)) < 0:
                    raise ConfigError(f"{where}: a mask of {mask['size']} keys keeping {mask.get('keep_first')}")
            if l.mlp is not None:
                mw = f"layers[{i}].mlp"
                _need(l.mlp, ("kind",), mw)
                if l.mlp["kind"] == "dense":
                    _need(l.mlp, ("ff",), mw)
                elif l.mlp["kind"] == "moe":
                    _need(l.mlp, ("expert", "router"), mw)
                    _need(l.mlp["expert"], ("ff",), mw + ".expert")
                    _need(l.mlp["router"], ("experts", "top"), mw + ".router")
                    r = l.mlp["router"]
                    if not 1 <= int(r["top"]) <= int(r["experts"]):
                        raise ConfigError(f"{mw}.router: top={r['top']} of {r['experts']} experts")
                else:
                    raise ConfigError(f"{mw}.kind={l.mlp['kind']!r} is not supported; known: dense, moe")
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
            "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale}, "layers": layers,
        }
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # --------------------------------------------------------------------- plan
    def _norm(self, name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"dim": self.width, "eps": self.norm_eps, "suffix": ""}, name)

    def _mixer(self, l: SameraxLayer) -> PartSpec:
        m = l.mixer
        rot = m.get("rot")
        if rot is not None and int(rot["dims"]) > 0:
            sc = rot.get("scaling")
            position = PartSpec("rotary", {
                "head_dim": int(m["dim"]), "rotary_dim": int(rot["dims"]), "theta": float(rot["base"]),
                "pairing": "halves", "table_precision": "float64",
                "scaling": {k: float(sc[k]) for k in ("factor", "original", "fast", "slow")} if sc else None})
        else:
            position = PartSpec("none", {})
        mask = m.get("mask")
        return PartSpec("differential_attention", {
            "hidden_size": self.width, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]),
            "map_dim": int(m["dim"]), "value_dim": int(m["vdim"]), "scale": float(m["scale"]),
            "diff": float(m["diff"]), "norm_eps": self.norm_eps, "bias": True,
            "window": int(mask["size"]) if mask is not None else None,
            "keep_first": int(mask.get("keep_first", 0)) if mask is not None else 0,
            "position": position,
        }, "mix.")

    def _feed_forward(self, l: SameraxLayer) -> Optional[PartSpec]:
        if l.mlp is None:
            return None
        if l.mlp["kind"] == "dense":
            return PartSpec("swiglu", {"hidden_size": self.width, "intermediate_size": int(l.mlp["ff"]),
                                       "names": ("gate", "up", "down")}, "mlp.")
        r = l.mlp["router"]
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "intermediate_size": int(l.mlp["expert"]["ff"]),
            "num_experts": int(r["experts"]), "num_identity": 0, "top": int(r["top"]),
            "router": "table", "vocab_size": self.vocab, "correction": False,
        }, "mlp.")

    def plan(self) -> ModelPlan:
        layers, order, index_of = [], [], {}
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
            layers.append(LayerSpec("pre_norm" if ff is not None else "pre_norm_mixer",
                                    f"l{i if j is None else j}.", norms, self._mixer(l), ff))
            order.append(RunEntry(index_of[i]))
        plan = ModelPlan(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": self.width,
                                             "suffix": "", "scale": self.embedding_scale}, "embed"),
            layers=tuple(layers), order=tuple(order),
            final_norm=self._norm("final.norm"),
            head=PartSpec("lm_head", {"hidden_size": self.width, "vocab_size": self.vocab, "tied_to": None,
                                      "suffix": "", "softcap": self.logit_softcap}, "head"),
        )
        plan.validate()
        return plan

    def describe(self) -> dict:
        return self.to_dict()
