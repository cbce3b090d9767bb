"""A short causal convolution over time, per channel, added to its own input:

    y_t = x_t + sum_j w[:, j] * x_(t - taps + 1 + j)          zeros in front of the sequence, no bias

It sits between a block's first norm and its mixer (category ``filter``).  The last taps-1 inputs of a sequence
are part of the request's state (a ``StateSpec`` slot of the run), so a prompt may be cut anywhere.  The sum is
formed in 32-bit from 32-bit inputs (the block hands the norm's rows over unrounded) and written in the engine's
type.  Kernel: the convolution of ``csrc/ssm.cu``.

Parameters: size (channels), taps, tensor (the weight's full name, [size, taps], the last column the current token's).
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..cache.spec import StateSpec
from ..ops import kernels as K
from ..weights.loader import WeightSpec
from .base import Part, register_part


class CausalConvFilter(Part):
    wants_float32_input = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.size = int(self.p("size"))
        self.taps = int(self.p("taps"))
        self.tensor = self.p("tensor", None) or self.name("weight")
        if not (1 <= self.taps <= 16):
            raise ValueError(f"{self.tensor}: {self.taps} taps (1 to 16)")
        self.weight = None

    def cache_spec(self):
        return StateSpec((max(1, (self.taps - 1) * self.size),), torch.float32)

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.tensor, (self.size, self.taps), as_float32=True)]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = self._vector32(tensors[self.tensor])

    def forward(self, x: torch.Tensor, ctx, slot: int) -> torch.Tensor:
        out = ctx.workspace.get("filter.out", (x.shape[0], self.size), ctx.dtype)
        K.causal_conv(x, 0, self.size, self.weight, None, ctx.state(slot), 0, ctx, out, add_input=True)
        return out


register_part("filter", "causal_conv_filter", CausalConvFilter)
