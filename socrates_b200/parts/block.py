"""How the parts of one layer are wired around the residual stream.

"pre_norm" is the reference's block (model/qwen/qwen_kv_paged.py:186-189):
x = x + mixer(norm_0(x)); x = x + feed_forward(norm_1(x)).  The additions happen
inside the next norm's kernel: each branch leaves its output pending on the stream
and the following norm (of this layer, the next layer, or the final one) folds it in.
"""

from __future__ import annotations

from typing import Dict, Mapping

import torch

from .base import ParamSpec, ResidualStream, build_part, register_part
from .norm import fold_and_norm


class PreNormBlock:
    def __init__(self, layer_spec):
        if len(layer_spec.norms) != 2:
            raise ValueError("a pre_norm block has two norms")
        pre = layer_spec.prefix
        self.norms = [build_part("norm", s, pre + s.name) for s in layer_spec.norms]
        self.mixer = build_part("mixer", layer_spec.mixer, pre + layer_spec.mixer.name)
        self.feed_forward = build_part("feed_forward", layer_spec.feed_forward,
                                       pre + layer_spec.feed_forward.name)

    def parts(self):
        return [*self.norms, self.mixer, self.feed_forward]

    def parameters(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = {}
        for p in self.parts():
            out.update(p.parameters())
        return out

    def bind(self, tensors: Mapping, dtype) -> None:
        for p in self.parts():
            p.bind(tensors, dtype)

    @property
    def supports_graph(self) -> bool:
        return all(getattr(p, "supports_graph", True) for p in self.parts())

    def cache_needs(self):
        fn = getattr(self.mixer, "cache_needs", None)
        return fn() if fn is not None else None

    def streamed_weights(self):
        """Weight matrices in the order in which forward() streams them (optional for a part)."""
        return [*getattr(self.mixer, "streamed_weights", list)(),
                *getattr(self.feed_forward, "streamed_weights", list)()]

    def forward(self, ctx, stream: ResidualStream, cache) -> None:
        h = self.norms[0].apply(ctx, stream)
        stream.pending = self.mixer.forward(ctx, h, cache)
        h = self.norms[1].apply(ctx, stream)
        stream.pending = self.feed_forward.forward(ctx, h)


register_part("arrangement", "pre_norm", lambda layer_spec, name="": PreNormBlock(layer_spec))


class PreNormMixerBlock(PreNormBlock):
    """A pre-norm layer without a feed-forward: x = x + mixer(norm_0(x))."""

    def __init__(self, layer_spec):
        if len(layer_spec.norms) != 1 or layer_spec.feed_forward is not None:
            raise ValueError("a pre_norm_mixer block has one norm and no feed-forward")
        pre = layer_spec.prefix
        self.norms = [build_part("norm", s, pre + s.name) for s in layer_spec.norms]
        self.mixer = build_part("mixer", layer_spec.mixer, pre + layer_spec.mixer.name)
        self.feed_forward = None

    def parts(self):
        return [*self.norms, self.mixer]

    def streamed_weights(self):
        return [*getattr(self.mixer, "streamed_weights", list)()]

    def forward(self, ctx, stream: ResidualStream, cache) -> None:
        h = self.norms[0].apply(ctx, stream)
        stream.pending = self.mixer.forward(ctx, h, cache)


register_part("arrangement", "pre_norm_mixer", lambda layer_spec, name="": PreNormMixerBlock(layer_spec))


class SandwichBlock:
    """A block that norms every branch on both sides:
    x = x + norm_1b(mixer(norm_1(x))); x = x + norm_2b(feed_forward(norm_2(x))).
    A layer without a feed-forward has the first half only (two norms instead of four).

    The norm after a branch costs no kernel of its own: the branch is left pending with
    the gain and eps of its norm, and the kernel that folds it into the residual (the
    next norm of this or the following layer, a stream op, or the final norm) norms the
    branch's sum first."""

    def __init__(self, layer_spec):
        want = 4 if layer_spec.feed_forward is not None else 2
        if len(layer_spec.norms) != want:
            raise ValueError(f"a sandwich block with{'' if want == 4 else 'out'} a feed-forward has {want} norms")
        pre = layer_spec.prefix
        self.norms = [build_part("norm", s, pre + s.name) for s in layer_spec.norms]
        self.mixer = build_part("mixer", layer_spec.mixer, pre + layer_spec.mixer.name)
        self.feed_forward = None
        if layer_spec.feed_forward is not None:
            self.feed_forward = build_part("feed_forward", layer_spec.feed_forward,
                                           pre + layer_spec.feed_forward.name)

    def parts(self):
        return [*self.norms, self.mixer, *([self.feed_forward] if self.feed_forward is not None else [])]

    def parameters(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = {}
        for p in self.parts():
            out.update(p.parameters())
        return out

    def bind(self, tensors: Mapping, dtype) -> None:
        for p in self.parts():
            p.bind(tensors, dtype)

    @property
    def supports_graph(self) -> bool:
        return all(getattr(p, "supports_graph", True) for p in self.parts())

    def cache_needs(self):
        fn = getattr(self.mixer, "cache_needs", None)
        return fn() if fn is not None else None

    def streamed_weights(self):
        return [*getattr(self.mixer, "streamed_weights", list)(),
                *(getattr(self.feed_forward, "streamed_weights", list)() if self.feed_forward is not None else [])]

    @staticmethod
    def _normed_on_entry(branch, norm):
        branch.post_gain, branch.post_eps = norm.gain, norm.eps
        return branch

    def forward(self, ctx, stream: ResidualStream, cache) -> None:
        h = self.norms[0].apply(ctx, stream)
        stream.pending = self._normed_on_entry(self.mixer.forward(ctx, h, cache), self.norms[1])
        if self.feed_forward is not None:
            h = self.norms[2].apply(ctx, stream)
            stream.pending = self._normed_on_entry(self.feed_forward.forward(ctx, h), self.norms[3])


register_part("arrangement", "sandwich_norm", lambda layer_spec, name="": SandwichBlock(layer_spec))


class BranchNormBlock(SandwichBlock):
    """A block that norms every branch on its way OUT only:
    x = x + norm_1(mixer(x)); x = x + norm_2(feed_forward(x)).
    Mixer and feed-forward read the stream itself.  A layer without a feed-forward has one norm.

    As in the sandwich block the norm after a branch rides with the pending branch and is applied by
    whoever folds it into the residual.  What a branch reads is the residual rounded to the model
    dtype, written by the same folding kernel (no gain: nothing is normed); the float32 engine reads
    the residual in place."""

    def __init__(self, layer_spec):
        want = 2 if layer_spec.feed_forward is not None else 1
        if len(layer_spec.norms) != want:
            raise ValueError(f"a branch_norm block with{'' if want == 2 else 'out'} a feed-forward has {want} norm(s)")
        pre = layer_spec.prefix
        self.norms = [build_part("norm", s, pre + s.name) for s in layer_spec.norms]
        self.mixer = build_part("mixer", layer_spec.mixer, pre + layer_spec.mixer.name)
        self.feed_forward = None
        if layer_spec.feed_forward is not None:
            self.feed_forward = build_part("feed_forward", layer_spec.feed_forward,
                                           pre + layer_spec.feed_forward.name)

    @staticmethod
    def _stream_rows(ctx, stream: ResidualStream) -> torch.Tensor:
        waiting = stream.pending is not None or stream.add_rows is not None or stream.add_vec is not None
        if ctx.dtype == torch.float32:
            if waiting:
                fold_and_norm(stream, None, None, 0.0)
            return stream.residual
        out = ctx.buffers.take("stream_rows", stream.residual.shape[0], (stream.residual.shape[1],), ctx.dtype)
        fold_and_norm(stream, None, out, 0.0)
        return out

    def forward(self, ctx, stream: ResidualStream, cache) -> None:
        h = self._stream_rows(ctx, stream)
        stream.pending = self._normed_on_entry(self.mixer.forward(ctx, h, cache), self.norms[0])
        if self.feed_forward is not None:
            h = self._stream_rows(ctx, stream)
            stream.pending = self._normed_on_entry(self.feed_forward.forward(ctx, h), self.norms[1])


register_part("arrangement", "branch_norm", lambda layer_spec, name="": BranchNormBlock(layer_spec))
