"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * g, eps inside the root.

The gain g is the stored tensor itself, or `offset` + the stored tensor for checkpoints
that keep their gains around zero (`offset` = 1: g = 1 + w; the sum is made once, in
float32, when the weights are bound).  The tensor is named `<name><suffix>` (suffix
"weight" unless the plan says otherwise).

The reference computes the norm in the activations' dtype (model/qwen/qwen_kv_cont.py:45-53);
here the sum of squares, the root and the product are float32 and only the result is
rounded to the model dtype.  The kernel also adds what is waiting on the stream to the
residual first: the pending branch (normed on its way in if the block says so), rows and
a vector that a stream op left.  That addition is the residual sum of the block.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..kernels import ops
from .base import ParamSpec, Part, ResidualStream, register_part


def fold_and_norm(stream: ResidualStream, gain: Optional[torch.Tensor], out: Optional[torch.Tensor],
                  eps: float, row_index: Optional[torch.Tensor] = None) -> None:
    """Add everything that waits on the stream to the residual and write the normed rows to `out`
    (None: only the residual moves on).  With `row_index` only those rows are computed and nothing
    on the stream changes."""
    b = stream.pending
    if stream.streams is not None or (b is not None and (b.scale != 1.0 or b.also is not None)):
        raise ValueError("several residual streams, a scaled branch or two branches side by side are folded by "
                         "the norms of parts/hyper.py; this norm takes the plain residual")
    plain = (b is None or b.plain) and stream.add_rows is None and stream.add_vec is None
    if plain and out is not None and gain is not None:
        ops.add_rmsnorm(stream.residual, b.partial if b is not None else None, gain, out, eps, row_index)
    else:
        ops.fold_rmsnorm(stream.residual, b.partial if b is not None else None, gain, out, eps, row_index,
                         branch_bias=b.bias if b is not None else None,
                         branch_gain=b.post_gain if b is not None else None,
                         branch_eps=b.post_eps if b is not None else 0.0,
                         add_rows=stream.add_rows, add_vec=stream.add_vec)
    if row_index is None:
        stream.pending = None
        stream.add_rows = stream.add_vec = None


class RMSNorm(Part):
    def __init__(self, spec, name):
        super().__init__(spec, name)
        self.dim = int(spec.params["dim"])
        self.eps = float(spec.params["eps"])
        self.offset = float(spec.params.get("offset", 0.0))
        self.tensor = self.name + str(spec.params.get("suffix", "weight"))
        self.gain: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        return {self.tensor: ParamSpec((self.dim,), role="gain", init="around_zero" if self.offset else "gain")}

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        g = tensors[self.tensor]
        self.gain = (g + self.offset).contiguous() if self.offset else g

    def apply(self, ctx, stream: ResidualStream, row_index: Optional[torch.Tensor] = None,
              buffer: str = "normed", out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """Fold what waits on the stream into the residual and return the normed rows.

        With `row_index` only those rows are normed (for the head) and the residual
        is left unchanged.
        """
        M = stream.residual.shape[0] if row_index is None else row_index.numel()
        take = ctx.buffers.take if row_index is None else ctx.buffers.take_wanted
        out = take(buffer, M, (self.dim,), out_dtype or ctx.dtype)
        fold_and_norm(stream, self.gain, out, self.eps, row_index)
        return out


register_part("norm", "rmsnorm", RMSNorm)
