"""Gated delta rule: a recurrent mixer. Per request and head it keeps a float32 matrix
S [head_dim, v_head_dim] and per token does, in this order,

    S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

with one decay g per (head, key channel), so the read-out sees the token's own write.
q and k (num_kv_heads x head_dim; head h uses q/k head h // (heads / kv_heads)) and v
(num_heads x v_head_dim) pass a short causal convolution per channel (`conv_taps` taps, the
last one the current token's, zeros before the start) and SiLU; q and k are then made unit
vectors per head (x / sqrt(sum x^2 + 1e-6)), q also times head_dim^-1/2. beta = sigmoid(W_b h);
g = exp(-exp(A_log) * softplus(W_a2 (W_a1 h) + dt_bias)); each head's o is divided by its root
mean square (`eps`), multiplied by a weight shared by the heads and by sigmoid(W_g2 (W_g1 h)),
and projected by W_o. Everything after the projections is float32 in both serving types.

The state slot of a request holds S for every head (transposed, [heads, v_head_dim,
head_dim]) and the convolutions' last taps - 1 inputs; the scheduler hands it out zeroed.
Three products feed the recurrence: q | k | v | beta in one, the first halves of the two
low-rank pairs in one, and their second halves in one (a block-diagonal matrix, whose zeros
add nothing); its result, the decay rates and gates before their activations, is float32. The
ranks of the pairs come from the spec (`decay_rank`, `gate_rank`).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..config.schema import ConfigError, PartSpec
from ..weights.loader import WeightSpec
from .base import Mixer, PositionEncoding, StateSpec, register_part
from .linear import linear, prepare_weight


class GatedDeltaRule(Mixer):
    def __init__(self, spec: PartSpec, hidden_size: int, position: Optional[PositionEncoding]):
        super().__init__(spec, hidden_size, position)
        self.heads, self.kv_heads = int(spec["num_heads"]), int(spec["num_kv_heads"])
        self.dk, self.dv = int(spec["head_dim"]), int(spec["v_head_dim"])
        self.taps = int(spec["conv_taps"])
        self.rank_a, self.rank_g = int(spec["decay_rank"]), int(spec["gate_rank"])
        self.eps = float(spec["eps"])
        if self.heads <= 0 or self.kv_heads <= 0 or self.heads % self.kv_heads:
            raise ConfigError(f"gated_delta: num_heads {self.heads} must be a positive multiple of num_kv_heads {self.kv_heads}")
        if not 0 < self.dk <= 256 or self.dv <= 0:
            raise ConfigError("gated_delta: head_dim must be between 1 and 256 and v_head_dim positive")
        if not 1 <= self.taps <= 16 or self.rank_a <= 0 or self.rank_g <= 0:
            raise ConfigError("gated_delta: conv_taps must be between 1 and 16 and the ranks positive")
        self.cq, self.cv = self.kv_heads * self.dk, self.heads * self.dv
        self.conv_channels = 2 * self.cq + self.cv
        self.conv_offset = self.heads * self.dk * self.dv
        widths = [("q", self.cq), ("k", self.cq), ("v", self.cv), ("b", self.heads)]
        self.offsets, at = {}, 0
        for name, width in widths:
            self.offsets[name] = at
            at += width
        self.proj_width = at
        self.w_in = self.w_low = self.w_rates = self.w_o = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        h = self.hidden_size
        return {
            "q": WeightSpec((self.cq, h)), "k": WeightSpec((self.cq, h)), "v": WeightSpec((self.cv, h)),
            "q.conv": WeightSpec((self.cq, self.taps), std=0.5), "k.conv": WeightSpec((self.cq, self.taps), std=0.5),
            "v.conv": WeightSpec((self.cv, self.taps), std=0.5),
            "b": WeightSpec((self.heads, h)), "A_log": WeightSpec((self.heads,), std=0.5),
            "norm": WeightSpec((self.dv,), init="norm", std=0.1),
            "a1": WeightSpec((self.rank_a, h)), "a2": WeightSpec((self.heads * self.dk, self.rank_a), std=0.2),
            "dt_bias": WeightSpec((self.heads * self.dk,), std=0.5),
            "g1": WeightSpec((self.rank_g, h)), "g2": WeightSpec((self.cv, self.rank_g), std=0.2),
            "o": WeightSpec((h, self.cv)),
        }

    def load(self, tensors, dtype):
        def stacked(names):
            parts = [tensors[n] for n in names]
            common = torch.float32 if any(p.dtype == torch.float32 for p in parts) else parts[0].dtype
            return torch.cat([p.to(common) for p in parts], dim=0).contiguous()
        self.w_in = prepare_weight(stacked(("q", "k", "v", "b")), dtype)
        self.w_low = prepare_weight(stacked(("a1", "g1")), dtype)
        a2, g2 = tensors["a2"], tensors["g2"]
        common = torch.float32 if torch.float32 in (a2.dtype, g2.dtype) else a2.dtype
        second = torch.zeros((a2.shape[0] + g2.shape[0], self.rank_a + self.rank_g), dtype=common, device=a2.device)
        second[: a2.shape[0], : self.rank_a] = a2
        second[a2.shape[0]:, self.rank_a:] = g2
        self.w_rates = prepare_weight(second, dtype)
        self.w_o = prepare_weight(tensors["o"], dtype)
        small = {n: tensors[n] for n in ("q.conv", "k.conv", "v.conv", "A_log", "dt_bias", "norm")}
        if len({t.dtype for t in small.values()}) > 1:
            small = {n: t.float() for n, t in small.items()}
        self.conv_w = torch.cat([small["q.conv"], small["k.conv"], small["v.conv"]], dim=0).contiguous()
        self.a_log, self.dt_bias = small["A_log"], small["dt_bias"]
        self.norm = small["norm"]

    def first_weight(self):
        return self.w_in

    def state_spec(self) -> StateSpec:
        size = self.conv_offset + (self.taps - 1) * self.conv_channels
        return StateSpec(((size + 3) // 4 * 4,), torch.float32)          # slots start on 16-byte boundaries

    def forward(self, ctx, x, cache, writes_cache: bool = True):
        if not writes_cache:
            raise ConfigError("gated_delta: a recurrent state cannot be shared between layer runs")
        proj = linear(ctx, x, self.w_in)
        rates = linear(ctx, linear(ctx, x, self.w_low), self.w_rates, out_dtype=torch.float32)
        q, k, v, beta, decay, gate = ops.delta_prep(
            proj, rates, self.offsets, kv_heads=self.kv_heads, heads=self.heads, dk=self.dk, dv=self.dv, taps=self.taps,
            conv_w=self.conv_w, a_log=self.a_log, dt_bias=self.dt_bias, state=cache.state,
            conv_offset=self.conv_offset, ctx=ctx)
        o = ops.delta_scan(q, k, v, beta, decay, cache.state, ctx, kv_heads=self.kv_heads, heads=self.heads,
                           dk=self.dk, dv=self.dv)
        y = ops.delta_out(o, gate, self.norm, self.eps, heads=self.heads, dv=self.dv, out_dtype=ctx.dtype)
        return linear(ctx, y, self.w_o, out_dtype=torch.float32)


register_part("mixer", "gated_delta", GatedDeltaRule, replace=True)
