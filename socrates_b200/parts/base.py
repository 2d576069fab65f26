"""Interfaces of the parts a model is put together from, and their registries.

A part is built from a `PartSpec` (its sizes and constants), declares the tensors it
needs by name, receives them once (`bind`), and then runs on the tokens of a step.
No part knows which model it sits in; which part a layer uses is decided layer by
layer by the plan.  The five kinds and what each must provide:

* **norm**           `apply(ctx, stream, row_index=None) -> normed [M, d]`: folds the
                     stream's pending branch output into the residual and norms it.
* **position**       `tables() -> (inv_freq float32 [rotary_dim/2], rotary_dim)`:
                     what the mixer's rotation kernel multiplies positions with.
* **mixer**          `cache_needs() -> CacheNeeds | None` and
                     `forward(ctx, x [N, d], cache: CacheView) -> Branch`.
* **feed_forward**   `forward(ctx, x [N, d]) -> Branch`.
* **arrangement**    `forward(ctx, stream, cache: CacheView)`: wires norms, mixer and
                     feed-forward of one layer around the residual stream.
* **stream_op**      `apply(ctx, stream)`: acts on the residual stream between layer runs
                     (named by `RunEntry.before`); `needs_embedding_output = True` makes the
                     model keep the embedding's output on the stream for it.

A `Branch` is the float32 output of a mixer or feed-forward as `S` partial sums
`[S, N, d]` (S > 1 when the last matrix product was split along K); the next norm
adds them to the residual in a fixed order, so the sum costs no pass of its own.

To add a part: subclass `Part`, give it `parameters()`, `bind()` and the method of
its kind, and call `register_part(kind_group, name, cls)`.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Mapping, Optional, Tuple

import torch

from ..config.plan import PartSpec


@dataclass(frozen=True)
class ParamSpec:
    """One tensor a part expects: its shape, and how random weights are drawn for it.

    role "matrix": a weight matrix, kept in the model dtype (bfloat16 or float32).
    role "gain":   a norm gain (or another small float32 parameter), always held as float32 on the device.
    role "int":    an integer table, int32 on the device.
    init "normal": N(0, 0.02); init "gain": 1 + N(0, 0.1); init "around_zero": N(0, 0.1);
    init "uniform": U(lo, hi) with `bounds` = (lo, hi); init "distinct" (role "int"): every row holds
    different integers from lo .. hi - 1.
    """
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"
    bounds: Tuple[float, float] = (0.0, 1.0)
    # A dim of -1 in `shape` is read from the file (a table whose length the configuration does
    # not give); `default_shape` is what random weights are drawn with then.
    default_shape: Optional[Tuple[int, ...]] = None

    def matches(self, shape) -> bool:
        shape = tuple(shape)
        return len(shape) == len(self.shape) and all(a == -1 or a == b for a, b in zip(self.shape, shape))

    @property
    def draw_shape(self) -> Tuple[int, ...]:
        return tuple(self.default_shape) if self.default_shape is not None else tuple(self.shape)


class Part:
    """Base of all parts.  `name` is the full checkpoint prefix of the part's tensors."""

    def __init__(self, spec: PartSpec, name: str):
        self.spec = spec
        self.name = name

    def parameters(self) -> Dict[str, ParamSpec]:
        """Full checkpoint name -> ParamSpec of every tensor this part reads."""
        return {}

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype) -> None:
        """Receive the tensors named by `parameters()`, already on the device."""

    supports_graph = True   # False if forward() needs host values that change per step


@dataclass
class Branch:
    """Float32 partial sums `[S, N, d]` waiting to be added to the residual.

    `bias` (float32 [d]) is added to their sum; with `post_gain` the sum is first normed
    (x / sqrt(mean(x^2) + post_eps) * post_gain) and joins the residual only then: a block
    that norms its branches on both sides sets these, and whoever folds the branch into the
    residual (the next norm's kernel) does the arithmetic.

    `scale` multiplies the sum (and its bias); `also` is a second branch that joins beside this
    one with a scale of its own (two mixers side by side).  Only the folding kernel of the
    residual streams (`parts/hyper.py`) takes these two."""
    partial: torch.Tensor
    bias: Optional[torch.Tensor] = None
    post_gain: Optional[torch.Tensor] = None
    post_eps: float = 0.0
    scale: float = 1.0
    also: Optional["Branch"] = None

    @property
    def plain(self) -> bool:
        return self.bias is None and self.post_gain is None and self.scale == 1.0 and self.also is None


class ResidualStream:
    """The float32 residual `[N, d]` of a step and the branch output not yet added."""

    def __init__(self, residual: torch.Tensor):
        self.residual = residual
        self.pending: Optional[Branch] = None
        # What else joins the residual at the next fold: float32 rows [N, d] and a vector [d].
        self.add_rows: Optional[torch.Tensor] = None
        self.add_vec: Optional[torch.Tensor] = None
        self.embedding_output: Optional[torch.Tensor] = None   # kept by the model when a stream op asks
        # Several residual streams (hyper-connections): float32 [N, s, d] once a block has made them
        # (`fresh`: they are still to be filled from `residual`), and how the pending branch joins
        # them: (mix [s, s], out weights [s], factor) left by the block that left the branch.
        self.streams: Optional[torch.Tensor] = None
        self.fresh = False
        self.joining = None


_REGISTRIES: Dict[str, Dict[str, Callable]] = {
    "norm": {}, "position": {}, "mixer": {}, "feed_forward": {}, "arrangement": {},
    "embedding": {}, "head": {}, "stream_op": {},
}


def register_part(group: str, kind: str, factory: Callable, *, replace: bool = False) -> None:
    """Make `factory(spec, name)` (or, for arrangements, `factory(layer_spec, parts...)`)
    available under `kind` in one of the groups above."""
    if group not in _REGISTRIES:
        raise KeyError(f"unknown part group {group!r}; known: {sorted(_REGISTRIES)}")
    if kind in _REGISTRIES[group] and not replace:
        raise ValueError(f"{group} kind {kind!r} is already registered")
    _REGISTRIES[group][kind] = factory


def unregister_part(group: str, kind: str) -> None:
    _REGISTRIES[group].pop(kind, None)


def build_part(group: str, spec: PartSpec, name: str):
    reg = _REGISTRIES[group]
    if spec.kind not in reg:
        raise KeyError(f"no {group} of kind {spec.kind!r}; known: {sorted(reg)}")
    return reg[spec.kind](spec, name)


def registered(group: str) -> list[str]:
    return sorted(_REGISTRIES[group])
