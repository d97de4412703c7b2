"""Generalized delta rule: a recurrent mixer whose state per request and head is a float32 matrix
S [head_dim, head_dim]. Per token, with the unit key u = k / sqrt(|k|^2 + 1e-6), a decay w and a
removal rate a per (head, key channel),

    S <- diag(w) S - (a * u) (u^T S) + k v^T      (both first terms read the old S);   o = S^T r

r, k, v = W_r h, W_k h, W_v h (num_heads x head_dim each);
w = exp(-exp(-1/2) * sigmoid(W_w2 tanh(W_w1 h) + w0)), a low-rank pair of rank `decay_rank` with a
tanh between its halves; a = sigmoid(W_a h + a.b). Each head's o is divided by its root mean
square (`eps`), multiplied by a weight `norm` [num_heads * head_dim] and by sigmoid(W_g h), and
projected by W_o. Everything after the projections is float32 in both serving types.

One product makes r | k | v | g | a | the low-rank pair's first half; the second half's product is
float32. The state slot of a request holds S for every head, transposed ([heads, value, key]); the
scheduler hands it out zeroed.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..config.schema import ConfigError, PartSpec
from ..weights.loader import WeightSpec
from .base import Mixer, PositionEncoding, StateSpec, register_part
from .linear import linear, prepare_weight


class GeneralDeltaRule(Mixer):
    def __init__(self, spec: PartSpec, hidden_size: int, position: Optional[PositionEncoding]):
        super().__init__(spec, hidden_size, position)
        self.heads, self.d = int(spec["num_heads"]), int(spec["head_dim"])
        self.rank, self.eps = int(spec["decay_rank"]), float(spec["eps"])
        if self.heads <= 0 or not 0 < self.d <= 256 or self.rank <= 0:
            raise ConfigError("general_delta: num_heads and decay_rank must be positive, head_dim between 1 and 256")
        self.width = self.heads * self.d
        self.offsets = {name: i * self.width for i, name in enumerate(("r", "k", "v", "g", "a"))}
        self.low_offset = 5 * self.width
        self.w_in = self.w_second = self.w_o = self.w0 = self.a_bias = self.norm = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        h, w = self.hidden_size, self.width
        specs = {name: WeightSpec((w, h)) for name in ("r", "k", "v", "g", "a")}
        specs.update({"a.b": WeightSpec((w,), std=0.5), "w1": WeightSpec((self.rank, h)),
                      "w2": WeightSpec((w, self.rank), std=0.2), "w0": WeightSpec((w,), std=0.5),
                      "norm": WeightSpec((w,), init="norm", std=0.1), "o": WeightSpec((h, w))})
        return specs

    def load(self, tensors, dtype):
        parts = [tensors[n] for n in ("r", "k", "v", "g", "a", "w1")]
        common = torch.float32 if any(p.dtype == torch.float32 for p in parts) else parts[0].dtype
        self.w_in = prepare_weight(torch.cat([p.to(common) for p in parts], dim=0).contiguous(), dtype)
        self.w_second = prepare_weight(tensors["w2"], dtype)
        self.w_o = prepare_weight(tensors["o"], dtype)
        small = {n: tensors[n] for n in ("w0", "a.b")}
        if len({t.dtype for t in small.values()}) > 1:
            small = {n: t.float() for n, t in small.items()}
        self.w0, self.a_bias, self.norm = small["w0"], small["a.b"], tensors["norm"]

    def first_weight(self):
        return self.w_in

    def state_spec(self) -> StateSpec:
        return StateSpec(((self.heads * self.d * self.d + 3) // 4 * 4,), torch.float32)

    def forward(self, ctx, x, cache, writes_cache: bool = True):
        if not writes_cache:
            raise ConfigError("general_delta: a recurrent state cannot be shared between layer runs")
        proj = linear(ctx, x, self.w_in)
        inner = linear(ctx, ops.tanh_columns(proj, self.low_offset, self.rank), self.w_second, out_dtype=torch.float32)
        r, k, v, decay, unit, removal, gate = ops.general_delta_prep(proj, inner, self.offsets, heads=self.heads, d=self.d,
                                                                     w0=self.w0, a_bias=self.a_bias)
        o = ops.general_delta_scan(r, k, v, decay, unit, removal, cache.state, ctx, heads=self.heads, d=self.d)
        y = ops.delta_out(o, gate, self.norm, self.eps, heads=self.heads, dv=self.d, out_dtype=ctx.dtype)
        return linear(ctx, y, self.w_o, out_dtype=torch.float32)


register_part("mixer", "general_delta", GeneralDeltaRule, replace=True)
