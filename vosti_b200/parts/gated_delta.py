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

A second form of the rule is chosen by parameters: `decay` = "head" keeps one decay per head
(`dt_bias` [heads]) instead of one per (head, key channel); ranks of 0 replace both low-rank pairs
by plain projections `a` [decay columns, hidden] and `g` [heads * v_head_dim, hidden] (one product,
float32 result); `gate_activation` = "silu" gates the output with z * sigmoid(z) instead of
sigmoid(z).
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
        self.rank_a, self.rank_g = int(spec.get("decay_rank", 0) or 0), int(spec.get("gate_rank", 0) or 0)
        self.eps = float(spec["eps"])
        decay, gate = spec.get("decay", "channel"), spec.get("gate_activation", "sigmoid")
        if decay not in ("channel", "head") or gate not in ("sigmoid", "silu"):
            raise ConfigError("gated_delta: decay is 'channel' or 'head', gate_activation 'sigmoid' or 'silu'")
        self.decay_per_head, self.gate_silu = decay == "head", gate == "silu"
        if (self.rank_a == 0) != (self.rank_g == 0):
            raise ConfigError("gated_delta: the decay and the gate are both low-rank pairs or both plain projections")
        if self.heads <= 0 or self.kv_heads <= 0 or self.heads % self.kv_heads:
            raise ConfigError(f"gated_delta: num_heads {self.heads} must be a positive multiple of num_kv_heads {self.kv_heads}")
        if not 0 < self.dk <= 256 or self.dv <= 0:
            raise ConfigError("gated_delta: head_dim must be between 1 and 256 and v_head_dim positive")
        if not 1 <= self.taps <= 16 or self.rank_a < 0 or self.rank_g < 0:
            raise ConfigError("gated_delta: conv_taps must be between 1 and 16 and the ranks not negative")
        self.decay_cols = self.heads if self.decay_per_head else self.heads * self.dk
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
        specs = {
            "q": WeightSpec((self.cq, h)), "k": WeightSpec((self.cq, h)), "v": WeightSpec((self.cv, h)),
            "q.conv": WeightSpec((self.cq, self.taps), std=0.5), "k.conv": WeightSpec((self.cq, self.taps), std=0.5),
            "v.conv": WeightSpec((self.cv, self.taps), std=0.5),
            "b": WeightSpec((self.heads, h)), "A_log": WeightSpec((self.heads,), std=0.5),
            "norm": WeightSpec((self.dv,), init="norm", std=0.1),
            "dt_bias": WeightSpec((self.decay_cols,), std=0.5),
            "o": WeightSpec((h, self.cv)),
        }
        if self.rank_a:
            specs.update({"a1": WeightSpec((self.rank_a, h)), "a2": WeightSpec((self.decay_cols, self.rank_a), std=0.2),
                          "g1": WeightSpec((self.rank_g, h)), "g2": WeightSpec((self.cv, self.rank_g), std=0.2)})
        else:
            specs.update({"a": WeightSpec((self.decay_cols, h)), "g": WeightSpec((self.cv, h))})
        return specs

    def load(self, tensors, dtype):
        def stacked(names):
            parts = [tensors[n] for n in names]
            common = torch.float32 if any(p.dtype == torch.float32 for p in parts) else parts[0].dtype
            return torch.cat([p.to(common) for p in parts], dim=0).contiguous()
        self.w_in = prepare_weight(stacked(("q", "k", "v", "b")), dtype)
        if self.rank_a:
            self.w_low = prepare_weight(stacked(("a1", "g1")), dtype)
            a2, g2 = tensors["a2"], tensors["g2"]
            common = torch.float32 if torch.float32 in (a2.dtype, g2.dtype) else a2.dtype
            second = torch.zeros((a2.shape[0] + g2.shape[0], self.rank_a + self.rank_g), dtype=common, device=a2.device)
            second[: a2.shape[0], : self.rank_a] = a2
            second[a2.shape[0]:, self.rank_a:] = g2
            self.w_rates = prepare_weight(second, dtype)
        else:
            self.w_low = None
            self.w_rates = prepare_weight(stacked(("a", "g")), dtype)
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
        rates = linear(ctx, x if self.w_low is None else linear(ctx, x, self.w_low), self.w_rates, out_dtype=torch.float32)
        q, k, v, beta, decay, gate = ops.delta_prep(
            proj, rates, self.offsets, kv_heads=self.kv_heads, heads=self.heads, dk=self.dk, dv=self.dv, taps=self.taps,
            conv_w=self.conv_w, a_log=self.a_log, dt_bias=self.dt_bias, state=cache.state,
            conv_offset=self.conv_offset, ctx=ctx, decay_per_head=self.decay_per_head, gate_silu=self.gate_silu)
        o = ops.delta_scan(q, k, v, beta, decay, cache.state, ctx, kv_heads=self.kv_heads, heads=self.heads,
                           dk=self.dk, dv=self.dv)
        y = ops.delta_out(o, gate, self.norm, self.eps, heads=self.heads, dv=self.dv, out_dtype=ctx.dtype)
        return linear(ctx, y, self.w_o, out_dtype=torch.float32)


register_part("mixer", "gated_delta", GatedDeltaRule, replace=True)
