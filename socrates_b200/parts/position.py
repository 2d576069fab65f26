"""Position encodings as data for the mixer's rotation kernel.

With `scaling` (factor, original, fast, slow) the frequencies are stretched for contexts longer
than the `original` one, dim by dim: a dim that turns more than `fast` times over the original
context keeps its frequency, one that turns fewer than `slow` times gets frequency / factor, the
dims between are blended linearly by their index; every cosine and sine is then multiplied by
`magnitude` = 0.1 ln(factor) + 1, which the rotation kernel takes as a constant.

A position encoding hands the mixer a float32 table `inv_freq[rotary_dim/2]` and the
number of leading dims that rotate; the kernel computes angle = float32(position) *
inv_freq[j] and pairs dim j with j + rotary_dim/2 (or, with `pairing: "neighbours"`, dim 2j
with dim 2j+1: `neighbours` says which).  Keys are stored rotated, so
positions are absolute and nothing else in the engine knows about the encoding.
Another encoding (a fraction of the dims, scaled frequencies, none at all) is another
table: register a class with `tables()`.

A mixer asks for its tables when its weights are bound, so that the copy from the host happens
then: a pageable host-to-device copy issued in the middle of a step, between kernels that were
launched with programmatic stream serialization, stalled for good in about one run in four of a
2,048-token first step (it never did with that launch attribute off, nor with the tables made
beforehand).  Nothing inside a step copies from pageable host memory.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from .base import Part, register_part


class Rotary(Part):
    """inv_freq_j = theta^(-2j/D), j < D/2, in float32 exactly as the reference builds
    it (model/qwen/qwen_kv_cont.py:56-64)."""

    def __init__(self, spec, name=""):
        super().__init__(spec, name)
        self.head_dim = int(spec.params["head_dim"])
        self.rotary_dim = int(spec.params.get("rotary_dim", self.head_dim))
        self.theta = float(spec.params["theta"])
        pairing = str(spec.params.get("pairing", "halves"))
        if pairing not in ("halves", "neighbours"):
            raise ValueError(f"pairing {pairing!r} is neither 'halves' nor 'neighbours'")
        self.neighbours = pairing == "neighbours"
        if self.rotary_dim % 2 or not 0 <= self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self._table: Optional[torch.Tensor] = None
        self._low: Optional[torch.Tensor] = None
        self.scaling = spec.params.get("scaling")
        self.magnitude = 1.0                    # on every cosine and sine
        if self.scaling:
            for key in ("factor", "original", "fast", "slow"):
                if key not in self.scaling:
                    raise ValueError(f"scaled rotation lacks {key!r}")
            if not float(self.scaling["factor"]) > 0:
                raise ValueError("the scaling factor must be positive")
            self.magnitude = 0.1 * math.log(float(self.scaling["factor"])) + 1.0

    def _scaled(self, f: torch.Tensor) -> torch.Tensor:
        """Blend of f and f / factor by dim index (float64 in, float64 out)."""
        sc, r = self.scaling, self.rotary_dim
        factor, original = float(sc["factor"]), float(sc["original"])

        def dim_of(turns: float) -> float:       # the (fractional) pair index that turns `turns` times
            return r * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))

        lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
        hi = min(math.ceil(dim_of(float(sc["slow"]))), r - 1)
        ramp = ((torch.arange(r // 2, dtype=torch.float64) - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        return f / factor * ramp + f * (1.0 - ramp)

    def inv_freq(self) -> torch.Tensor:
        r = self.rotary_dim
        if self.scaling:
            exact = float(self.theta) ** (-torch.arange(0, r, 2, dtype=torch.float64) / r)
            return self._scaled(exact).float()
        if self.spec.params.get("table_precision") == "float64":
            # theta^(-2j/r) in double precision, rounded once to float32
            return (float(self.theta) ** (-torch.arange(0, r, 2, dtype=torch.float64) / r)).float()
        return 1.0 / (self.theta ** (torch.arange(0, r, 2).float() / r))

    def low_table(self, device) -> Optional[torch.Tensor]:
        """With `table_precision` float64: what rounding to float32 took from each frequency, as float32 (a
        kernel that carries its angles in two terms adds position * this); None otherwise."""
        if self.spec.params.get("table_precision") != "float64" or not self.rotary_dim or self.scaling:
            return None
        if self._low is None or self._low.device != torch.device(device):
            r = self.rotary_dim
            exact = float(self.theta) ** (-torch.arange(0, r, 2, dtype=torch.float64) / r)
            self._low = (exact - exact.float().double()).float().to(device).contiguous()
        return self._low

    def tables(self, device) -> Tuple[torch.Tensor, int]:
        if self._table is None or self._table.device != torch.device(device):
            t = self.inv_freq() if self.rotary_dim else torch.zeros(1)
            self._table = t.to(device=device, dtype=torch.float32).contiguous()
        return self._table, self.rotary_dim


class NoPosition(Part):
    """No rotation: the mixer's kernel passes every dim through."""

    neighbours = False
    magnitude = 1.0

    def __init__(self, spec, name=""):
        super().__init__(spec, name)
        self._table = None

    def tables(self, device):
        if self._table is None:
            self._table = torch.zeros(1, dtype=torch.float32, device=device)
        return self._table, 0


register_part("position", "rotary", Rotary)
register_part("position", "none", NoPosition)
