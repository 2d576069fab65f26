"""Mixers made of mixers.

"normed_mean": several mixers read the same input side by side; each output is RMS-normed
over the model width with a plain gain of its own and the results are averaged:
    out = (1 / n) * sum_i unit_rms(mixer_i(x)) * gain_i
Each inner mixer is an ordinary registered mixer built from its own spec; its tensors sit
under `<name><prefix_i>`, its gain is the tensor `<name><prefix_i>out`, and what it asks of
the cache (pages, state slots) is passed through with the prefix in front of state names.
The norms, the gains and the mean are one kernel that reads the inner products' partial sums.

"scaled_sum": two mixers read the same input side by side and their outputs are added with a constant each:
    out = scale_0 * mixer_0(x) + scale_1 * mixer_1(x)
Nothing is computed here: the second branch rides with the first (`Branch.also`) and the kernel that folds
the branch into the residual streams adds both, each with its scale.  Tensors and cache needs as above.
"""

from __future__ import annotations

from typing import Dict, List, Mapping

import torch

from ..cache.manager import CacheNeeds
from ..kernels import ops
from .base import Branch, ParamSpec, Part, build_part, register_part


class _SideBySide(Part):
    """Two inner mixers built from their own specs; tensors, graphs and cache needs passed through."""
    out_buffer = "branch"

    def __init__(self, spec, name):
        super().__init__(spec, name)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.prefixes: List[str] = [str(s.name) for s in p["branches"]]
        self.inner = [build_part("mixer", s, name + s.name) for s in p["branches"]]
        if len(self.inner) != 2:
            raise ValueError("two branches run side by side")
        for i, m in enumerate(self.inner):
            m.out_buffer = f"branch.{i}"

    def parameters(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = {}
        for m in self.inner:
            out.update(m.parameters())
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        for m in self.inner:
            m.bind(tensors, dtype)

    @property
    def supports_graph(self) -> bool:
        return all(getattr(m, "supports_graph", True) for m in self.inner)

    def cache_needs(self) -> CacheNeeds:
        paged, state = None, {}
        for pre, m in zip(self.prefixes, self.inner):
            n = m.cache_needs() if hasattr(m, "cache_needs") else None
            if n is None:
                continue
            if n.paged is not None:
                if paged is not None:
                    raise ValueError("only one mixer of a group can keep pages")
                paged = n.paged
            for key, s in n.state_specs().items():
                state[pre + key] = s
        return CacheNeeds(paged=paged, state=state or None)

    def streamed_weights(self):
        return [w for m in self.inner for w in getattr(m, "streamed_weights", list)()]


class NormedMean(_SideBySide):
    def __init__(self, spec, name):
        super().__init__(spec, name)
        self.eps = float(spec.params["eps"])
        self.gains = None

    def parameters(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = {}
        for pre, m in zip(self.prefixes, self.inner):
            out.update(m.parameters())
            out[self.name + pre + "out"] = ParamSpec((self.hidden,), role="gain", init="gain")
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        super().bind(tensors, dtype)
        self.gains = [tensors[self.name + pre + "out"] for pre in self.prefixes]

    def forward(self, ctx, x: torch.Tensor, cache) -> Branch:
        N = x.shape[0]
        parts = [m.forward(ctx, x, cache.sub(pre)) for pre, m in zip(self.prefixes, self.inner)]
        if not all(b.plain for b in parts):
            raise ValueError("an inner mixer's branch must be plain partial sums")
        out = ctx.buffers.take_flat(self.out_buffer, N * self.hidden, torch.float32).view(1, N, self.hidden)
        ops.normed_mean(out[0], parts[0].partial, self.gains[0], parts[1].partial, self.gains[1], self.eps,
                        1.0 / len(parts))
        return Branch(out)


register_part("mixer", "normed_mean", NormedMean)


class ScaledSum(_SideBySide):
    """Inner mixers that can take their projections from outside (`shared_projection = True`: their input
    projections are one `Linear` named `proj`, and `forward` accepts `proj=(matrix, first column)`) share ONE
    matrix product: the two weight matrices are laid one under the other when the weights are bound."""

    def __init__(self, spec, name):
        super().__init__(spec, name)
        self.scales = [float(v) for v in spec.params["scales"]]
        if len(self.scales) != 2:
            raise ValueError("a scale for each of the two branches")
        self.fused = None
        self.columns = [0, 0]

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        super().bind(tensors, dtype)
        if all(getattr(m, "shared_projection", False) for m in self.inner):
            from .linear import Linear
            self.columns = [0, self.inner[0].proj.out_features]
            self.fused = Linear(torch.cat([m.proj.weight for m in self.inner], dim=0))
            for m in self.inner:
                m.proj = None                    # the rows live in the shared matrix now

    def streamed_weights(self):
        if self.fused is None:
            return super().streamed_weights()
        return [self.fused.weight, *[m.o.weight for m in self.inner]]

    def forward(self, ctx, x: torch.Tensor, cache) -> Branch:
        if self.fused is not None:
            proj = self.fused(ctx, x, "side_proj")
            first, second = (m.forward(ctx, x, cache.sub(pre), proj=(proj, col))
                             for pre, m, col in zip(self.prefixes, self.inner, self.columns))
        else:
            first, second = (m.forward(ctx, x, cache.sub(pre)) for pre, m in zip(self.prefixes, self.inner))
        for b in (first, second):
            if b.also is not None or b.post_gain is not None or b.scale != 1.0:
                raise ValueError("an inner mixer's branch must be partial sums (and a bias, for the first)")
        if second.bias is not None:
            raise ValueError("only the first of two branches side by side may bring a bias")
        first.scale, second.scale = self.scales
        first.also = second
        return first


register_part("mixer", "scaled_sum", ScaledSum)
