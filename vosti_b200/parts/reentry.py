"""What happens to the residual stream where a pass of a layer loop begins.

'concat_linear': x <- W [x ; x0], one product of the stream (with whatever was still to be
added to it) beside the embedding output x0, with W [width, 2 * width] (x's columns first).
The result is the new float32 stream.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..config.schema import PartSpec
from ..weights.loader import WeightSpec
from .base import Part, register_part
from .linear import linear, prepare_weight


class ConcatReentry(Part):
    def __init__(self, spec: PartSpec, hidden_size: int):
        super().__init__(spec, hidden_size)
        self.weight = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"weight": WeightSpec((self.hidden_size, 2 * self.hidden_size))}

    def load(self, tensors, dtype):
        self.weight = prepare_weight(tensors["weight"], dtype)

    def forward(self, ctx, hidden, residual, first):
        """(hidden, residual) as a block would receive them, and the embedding output `first`;
        returns the same pair after the re-entry: nothing left to add, a new stream."""
        packed = ops.stream_sum(residual, hidden, out_dtype=ctx.dtype, tail=first)
        return None, linear(ctx, packed, self.weight, out_dtype=torch.float32)


register_part("reentry", "concat_linear", ConcatReentry, replace=True)
