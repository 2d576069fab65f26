"""Several residual streams instead of one (hyper-connections), and the layer norm that reads them.

Instead of one residual x a model keeps `s` streams x_1 .. x_s, all equal to the embedding's output at
first.  A sublayer (1: the mixer, 2: the feed-forward) with tensors `<layer>hc<q>.in [s]`, `.out [s]`,
`.mix [s, s]` reads and writes them so:

    u = sum_t in[t] x_t ;  y = sublayer(norm(u)) ;  x_t <- sum_f mix[f, t] x_f + m * out[t] * y     (all t at once)

with m a constant of the model; the model's output is the sum of the streams.  With `streams` absent the
block is the ordinary x <- x + m * sublayer(norm(x)).

Nothing of this is a kernel of its own: a sublayer leaves its output pending on the stream together with
how it joins (`stream.joining`), and the NEXT norm's kernel updates all streams, forms the next reading u
and norms it in one pass over the row (`ops.hyper_fold_norm`), as the other blocks' norms add the pending
branch to the one residual.  Streams, the update, the reading and the norm are float32.

"layernorm": y = (x - mean) / sqrt(mean((x - mean)^2) + eps) * w, no bias, float32, the variance taken
over the deviations.  It is the norm that folds the streams; on a plain residual it folds a pending branch
(also a scaled one, or two side by side) like the RMS norm does.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..kernels import ops
from .base import ParamSpec, Part, ResidualStream, build_part, register_part


def fold_streams(ctx, stream: ResidualStream, gain: Optional[torch.Tensor], eps: float, center: bool,
                 out: Optional[torch.Tensor], row_index: Optional[torch.Tensor] = None,
                 read: Optional[torch.Tensor] = None, read_out: Optional[torch.Tensor] = None,
                 keep: bool = False) -> None:
    """Join what waits on the stream (the pending branch, as `stream.joining` says), read the streams with
    `read` (None: their plain sum) and norm the reading into `out`.  With `row_index`, or with `keep`,
    nothing on the stream changes."""
    if stream.add_rows is not None or stream.add_vec is not None:
        raise ValueError("rows or a vector left by a stream op are not folded by this norm")
    b = stream.pending
    if b is not None and b.post_gain is not None:
        raise ValueError("a branch that is normed on its way in is not folded by this norm")
    mix, out_w, mult = stream.joining if stream.joining is not None else (None, None, 1.0)
    also = b.also if b is not None else None
    if also is not None and (also.bias is not None or also.also is not None or also.post_gain is not None):
        raise ValueError("the second of two branches side by side brings partial sums and a scale only")
    target = stream.streams if stream.streams is not None else stream.residual
    view_only = row_index is not None or keep
    if view_only and row_index is None:
        # every row, but nothing written: the kernel leaves the streams alone for a row index
        row_index = _all_rows(ctx, target.shape[0])
    ops.hyper_fold_norm(
        target, stream.residual if (stream.streams is not None and stream.fresh) else None,
        b.partial if b is not None else None, b.scale if b is not None else 1.0,
        also.partial if also is not None else None, also.scale if also is not None else 1.0,
        b.bias if b is not None else None, mix, out_w, mult, read, gain, eps, center, out, row_index, read_out)
    if not view_only:
        stream.pending = None
        stream.joining = None
        stream.fresh = False


def _all_rows(ctx, n: int) -> torch.Tensor:
    rows = ctx.buffers.take_flat("all_rows", ctx.buffers.max_rows, torch.int32)
    if not getattr(ctx.buffers, "_all_rows_filled", False):
        rows.copy_(torch.arange(ctx.buffers.max_rows, dtype=torch.int32, device=rows.device))
        ctx.buffers._all_rows_filled = True
    return rows[:n]


def settled_sum(ctx, stream: ResidualStream) -> torch.Tensor:
    """The residual as it stands with everything pending joined: float32 [N, d], the sum of the streams.
    For inspection (a hook after a layer run); nothing on the stream changes."""
    target = stream.streams if stream.streams is not None else stream.residual
    N, d = target.shape[0], target.shape[-1]
    out = torch.empty((N, d), dtype=torch.float32, device=target.device)
    fold_streams(ctx, stream, None, 0.0, False, None, read_out=out, keep=True)
    return out


class LayerNorm(Part):
    def __init__(self, spec, name):
        super().__init__(spec, name)
        self.dim = int(spec.params["dim"])
        self.eps = float(spec.params["eps"])
        self.center = bool(spec.params.get("center", True))     # False: an RMS norm that folds streams
        self.tensor = self.name + str(spec.params.get("suffix", "weight"))
        self.gain: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        return {self.tensor: ParamSpec((self.dim,), role="gain", init="gain")}

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        self.gain = tensors[self.tensor]

    def apply(self, ctx, stream: ResidualStream, row_index: Optional[torch.Tensor] = None,
              buffer: str = "normed", out_dtype: Optional[torch.dtype] = None,
              read: Optional[torch.Tensor] = None) -> torch.Tensor:
        target = stream.streams if stream.streams is not None else stream.residual
        M = target.shape[0] if row_index is None else row_index.numel()
        take = ctx.buffers.take if row_index is None else ctx.buffers.take_wanted
        out = take(buffer, M, (self.dim,), out_dtype or ctx.dtype)
        fold_streams(ctx, stream, self.gain, self.eps, self.center, out, row_index, read)
        return out


register_part("norm", "layernorm", LayerNorm)


class HyperConnectionBlock:
    """x_t <- sum_f mix[f, t] x_f + m * out[t] * sublayer(norm(sum_t in[t] x_t)) for the mixer and then the
    feed-forward (absent: the mixer only).  `streams` 0: one residual, x <- x + m * sublayer(norm(x)), and no
    tensors of its own.  The norms must be of a kind that folds streams ("layernorm")."""

    def __init__(self, layer_spec):
        self.s = int(layer_spec.params.get("streams", 0) or 0)
        self.mult = float(layer_spec.params.get("residual_mult", 1.0))
        self.hidden = int(layer_spec.params["hidden_size"])
        want = 2 if layer_spec.feed_forward is not None else 1
        if len(layer_spec.norms) != want:
            raise ValueError(f"a hyper-connection block with{'' if want == 2 else 'out'} a feed-forward has {want} norm(s)")
        if not 0 <= self.s <= 8:
            raise ValueError(f"{self.s} residual streams; the folding kernel takes up to 8")
        pre = layer_spec.prefix
        self.prefix = pre
        self.norms = [build_part("norm", s, pre + s.name) for s in layer_spec.norms]
        for n in self.norms:
            if not isinstance(n, LayerNorm):
                raise ValueError("the norms of a hyper-connection block must fold streams (kind 'layernorm')")
        self.mixer = build_part("mixer", layer_spec.mixer, pre + layer_spec.mixer.name)
        self.feed_forward = None
        if layer_spec.feed_forward is not None:
            self.feed_forward = build_part("feed_forward", layer_spec.feed_forward, pre + layer_spec.feed_forward.name)
        self.names = [f"{pre}hc{q + 1}." for q in range(want)]
        self.hc = [None] * want            # (in, out, mix) per sublayer

    def parts(self):
        return [*self.norms, self.mixer, *([self.feed_forward] if self.feed_forward is not None else [])]

    def parameters(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = {}
        for p in self.parts():
            out.update(p.parameters())
        if self.s:
            for n in self.names:
                out[n + "in"] = ParamSpec((self.s,), role="gain", init="uniform", bounds=(0.1, 0.6))
                out[n + "out"] = ParamSpec((self.s,), role="gain", init="uniform", bounds=(0.3, 1.0))
                out[n + "mix"] = ParamSpec((self.s, self.s), role="gain", init="uniform", bounds=(-0.1, 0.5))
        return out

    def bind(self, tensors: Mapping, dtype) -> None:
        for p in self.parts():
            p.bind(tensors, dtype)
        if self.s:
            self.hc = [(tensors[n + "in"], tensors[n + "out"], tensors[n + "mix"]) for n in self.names]

    @property
    def supports_graph(self) -> bool:
        return all(getattr(p, "supports_graph", True) for p in self.parts())

    def cache_needs(self):
        fn = getattr(self.mixer, "cache_needs", None)
        return fn() if fn is not None else None

    def streamed_weights(self):
        return [*getattr(self.mixer, "streamed_weights", list)(),
                *(getattr(self.feed_forward, "streamed_weights", list)() if self.feed_forward is not None else [])]

    def _leave(self, stream: ResidualStream, branch, q: int) -> None:
        stream.pending = branch
        if self.s:
            _, out_w, mix = self.hc[q]
            stream.joining = (mix, out_w, self.mult)
        else:
            stream.joining = (None, None, self.mult)

    def forward(self, ctx, stream: ResidualStream, cache) -> None:
        if self.s and stream.streams is None:
            # the first block of the model: every stream starts as the embedding's output
            if stream.pending is not None:
                raise ValueError("a branch is pending on a residual that is about to become several streams")
            stream.streams = ctx.buffers.take("streams", stream.residual.shape[0], (self.s, self.hidden), torch.float32)
            stream.fresh = True
        elif not self.s and stream.streams is not None:
            raise ValueError("a block with one residual follows a block with several streams")
        h = self.norms[0].apply(ctx, stream, read=self.hc[0][0] if self.s else None)
        self._leave(stream, self.mixer.forward(ctx, h, cache), 0)
        if self.feed_forward is not None:
            h = self.norms[1].apply(ctx, stream, read=self.hc[1][0] if self.s else None)
            self._leave(stream, self.feed_forward.forward(ctx, h), 1)


register_part("arrangement", "hyper_connections", lambda layer_spec, name="": HyperConnectionBlock(layer_spec))
