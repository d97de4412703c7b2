"""A per-layer token input: a gate computed from the stream picks from a small vector that belongs
to the token id, and the result is projected back to the model width and normed:

    e = table[tok][offset : offset + dim];   g = gelu_tanh(W_gate x) * e;   y = W_proj g;
    out = y / sqrt(mean(y^2) + eps) * norm

with gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))). `out` is float32 and is
added to the stream by whoever reads the stream next. The table [vocab, layers * dim] is one
tensor for the whole model, owned and published by the embedding part (`ctx.extras["token_table"]`,
ids in `ctx.extras["token_ids"]`); a layer reads its own `dim` columns from `offset` on.
Parameters: dim, offset, eps. Tensors: gate [dim, hidden], proj [hidden, dim], norm [hidden]
(a plain weight)."""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..config.schema import ConfigError, PartSpec
from ..weights.loader import WeightSpec
from .base import TokenInput, register_part
from .linear import linear, prepare_weight


class GatedTokenInput(TokenInput):
    def __init__(self, spec: PartSpec, hidden_size: int):
        super().__init__(spec, hidden_size)
        self.dim, self.offset, self.eps = int(spec["dim"]), int(spec["offset"]), float(spec["eps"])
        if self.dim <= 0 or self.offset < 0:
            raise ConfigError("gated_table: dim must be positive and offset non-negative")
        self.w_gate = self.w_proj = self.norm = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        h = self.hidden_size
        return {"gate": WeightSpec((self.dim, h)), "proj": WeightSpec((h, self.dim)),
                "norm": WeightSpec((h,), init="norm", std=0.1)}

    def load(self, tensors, dtype):
        self.w_gate, self.w_proj = prepare_weight(tensors["gate"], dtype), prepare_weight(tensors["proj"], dtype)
        self.norm = tensors["norm"]

    def first_weight(self):
        return self.w_gate

    def forward(self, ctx, x):
        table, ids = ctx.extras.get("token_table"), ctx.extras.get("token_ids")
        if table is None or ids is None:
            raise ConfigError("gated_table: the model's embedding publishes no table of per-token vectors")
        if self.offset + self.dim > table.shape[1]:
            raise ConfigError("gated_table: the layer's columns lie beyond the table")
        gate = ops.token_gate(linear(ctx, x, self.w_gate), ids, table, self.offset)
        y = linear(ctx, gate, self.w_proj, out_dtype=torch.float32)
        return ops.rms_stream(y, self.norm, self.eps, torch.float32)


register_part("token_input", "gated_table", GatedTokenInput, replace=True)
