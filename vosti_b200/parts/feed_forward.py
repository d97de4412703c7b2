"""Gated feed-forward with SiLU: down( silu(gate(x)) * up(x) ).

gate and up are one [2I, hidden] matrix (gate rows first) so that the projection is a
single product, as the reference's loader concatenates them
(python/vosti_kernels/model_families/qwen3/loader.py:55-58); the activation is
gate * sigmoid(gate) * up in float32 (kernels/triton_kernels/silu_mul.py:66-87).

Parameters besides `intermediate_size`: `tensor_names`, the checkpoint's names of the gate, up
and down matrices (default: Qwen3's), and `float32_out`, for models whose residual stream is
float32: the down projection is then not rounded to the serving type.

`ExpertMixture` is the same feed-forward as `experts` small ones, of which each token uses
the `top` with the largest router logits, weighted by the softmax over the chosen logits only.
Its experts may also be plain two-matrix feed-forwards, down(gelu(up(x))) with the exact (erf)
GELU, and its weights the chosen experts' shares of a softmax over all experts, divided by
their sum and multiplied by a constant.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..config.schema import ConfigError, PartSpec
from ..weights.loader import WeightSpec
from .base import FeedForward, register_part
from .linear import linear, prepare_weight, uses_tensor_cores


def stack_gate_up(gate: torch.Tensor, up: torch.Tensor, dtype: torch.dtype):
    """One [2I, hidden] matrix for the gate and up projections, and whether SiLU(gate)*up can be
    the tensor-core product's epilogue. If so, rows are laid out as blocks of 16 gate rows
    followed by their 16 up rows, so that both halves of an output land in one warp's slice of
    the accumulator; else the gate rows come first."""
    inter = gate.shape[0]
    common = torch.float32 if torch.float32 in (gate.dtype, up.dtype) else gate.dtype
    stacked = torch.cat([gate.to(common), up.to(common)], dim=0)
    fused = dtype == torch.bfloat16 and inter % 16 == 0 and uses_tensor_cores(dtype, stacked)
    if not fused:
        return stacked.contiguous(), False
    h = stacked.shape[1]
    blocks = torch.stack([stacked[:inter].view(-1, 16, h), stacked[inter:].view(-1, 16, h)], dim=1)
    return prepare_weight(blocks.reshape(2 * inter, h).contiguous(), dtype), True


def gated_activation(ctx, x, w_gate_up, fused: bool):
    if fused:
        return ops.gemm_tc(ops.materialize(x), w_gate_up, ctx.status, swiglu=True)
    return ops.silu_mul(linear(ctx, x, w_gate_up))


class SwiGLU(FeedForward):
    def __init__(self, spec: PartSpec, hidden_size: int):
        super().__init__(spec, hidden_size)
        self.inter = int(spec["intermediate_size"])
        if self.inter <= 0:
            raise ConfigError("swiglu: intermediate_size must be positive")
        self.names = tuple(spec.get("tensor_names") or ("gate_proj.weight", "up_proj.weight", "down_proj.weight"))
        self.float32_out = bool(spec.get("float32_out", False))
        self.w_gate_up = self.w_down = None
        self.fused = False

    def weight_specs(self) -> Dict[str, WeightSpec]:
        h, i = self.hidden_size, self.inter
        gate, up, down = self.names
        return {gate: WeightSpec((i, h)), up: WeightSpec((i, h)), down: WeightSpec((h, i))}

    def load(self, tensors, dtype):
        gate, up, down = self.names
        self.w_down = prepare_weight(tensors[down], dtype)
        self.w_gate_up, self.fused = stack_gate_up(tensors[gate], tensors[up], dtype)

    def first_weight(self):
        return self.w_gate_up

    def forward(self, ctx, x):
        mlp = gated_activation(ctx, x, self.w_gate_up, self.fused)
        if self.float32_out:
            return linear(ctx, mlp, self.w_down, out_dtype=torch.float32)
        return linear(ctx, mlp, self.w_down, allow_partial=True)     # summed by the norm that follows


register_part("feed_forward", "swiglu", SwiGLU, replace=True)


class ExpertMixture(FeedForward):
    """Parameters: experts, top, intermediate_size (of one expert), `float32_out`. Tensors:
    `router` [experts, hidden] and `e<i>.gate`, `e<i>.up`, `e<i>.down`. Further parameters:
    `gated` (default true; false: experts are down(gelu(up(x))), no `gate` tensors), `route`
    ("top_softmax", the default: softmax over the chosen logits; "softmax_renorm": softmax over
    all experts, the chosen scores divided by their sum + 1e-20) and `scale`, a constant on the
    weights (default 1).

    The router's logits are float32. The experts' gate and up matrices stand side by side as one
    [2 * experts * I, hidden] matrix and their down matrices as one [hidden, experts * I]: every
    token's activation is computed for all experts by one product, each expert's slice is
    multiplied by the token's weight for it (zero if it was not chosen), and one more product
    sums the chosen experts' outputs. No launch depends on the router's choice, so a step may be
    replayed from a CUDA graph.

    A step that brings portions of prompts (`GROUPED_FROM` tokens or more, not all of them single
    tokens; such a step is never recorded as a graph) takes another way, in which no expert
    computes a token that did not choose it: the (token, pick) pairs are sorted by expert on the
    device, the host reads how many each expert got (one synchronisation), every expert with
    work multiplies its run of gathered rows, and a last kernel adds every token's picks in pick
    order. The experts' gate and up matrices are kept a second time for it, one per expert."""

    GROUPED_FROM = 256

    def __init__(self, spec: PartSpec, hidden_size: int):
        super().__init__(spec, hidden_size)
        self.experts, self.top = int(spec["experts"]), int(spec["top"])
        self.inter = int(spec["intermediate_size"])
        self.float32_out = bool(spec.get("float32_out", False))
        self.gated = bool(spec.get("gated", True))
        self.route, self.scale = spec.get("route", "top_softmax"), float(spec.get("scale", 1.0))
        if self.experts <= 0 or not 0 < self.top <= self.experts or self.inter <= 0:
            raise ConfigError("moe: experts, top (at most experts) and intermediate_size must be positive")
        if self.route not in ("top_softmax", "softmax_renorm") or self.scale != self.scale:
            raise ConfigError("moe: route is 'top_softmax' or 'softmax_renorm' and scale a number")
        self.router = self.w_gate_up = self.w_down = None
        self.fused = False

    def weight_specs(self) -> Dict[str, WeightSpec]:
        h, i = self.hidden_size, self.inter
        specs = {"router": WeightSpec((self.experts, h), std=0.5)}
        for e in range(self.experts):
            specs.update({f"e{e}.up": WeightSpec((i, h)), f"e{e}.down": WeightSpec((h, i))})
            if self.gated:
                specs[f"e{e}.gate"] = WeightSpec((i, h))
        return specs

    def load(self, tensors, dtype):
        self.router = tensors["router"].float().contiguous()        # 32-bit logits from exact 32-bit products
        up = torch.cat([tensors[f"e{e}.up"] for e in range(self.experts)], dim=0)
        if self.gated:
            gate = torch.cat([tensors[f"e{e}.gate"] for e in range(self.experts)], dim=0)
            self.w_gate_up, self.fused = stack_gate_up(gate, up, dtype)
        else:
            self.w_gate_up, self.fused = prepare_weight(up.contiguous(), dtype), False
        self.w_down = prepare_weight(torch.cat([tensors[f"e{e}.down"] for e in range(self.experts)], dim=1).contiguous(), dtype)
        self.per_expert = []
        if self.top < self.experts:
            for e in range(self.experts):
                if self.gated:
                    gate_up, fused = stack_gate_up(tensors[f"e{e}.gate"], tensors[f"e{e}.up"], dtype)
                else:
                    gate_up, fused = prepare_weight(tensors[f"e{e}.up"], dtype), False
                self.per_expert.append((gate_up, fused, prepare_weight(tensors[f"e{e}.down"], dtype)))

    def first_weight(self):
        return self.w_gate_up

    def _activation(self, ctx, x, w_first, fused, dense=None):
        """An expert's (or all experts') hidden activation, times the dense weights if given."""
        if self.gated:
            act = gated_activation(ctx, x, w_first, fused)
            return act if dense is None else ops.moe_scale(act, dense, self.inter)
        return ops.moe_scale(ops.materialize(linear(ctx, x, w_first)), dense, self.inter, gelu=True)

    def _grouped(self, ctx, x, chosen, weights):
        offsets, rows, where = ops.moe_group(chosen, self.experts)
        gathered = ops.gather_rows(x, rows, ctx.status)
        bounds = offsets.tolist()                      # the host learns the experts' shares here
        y = torch.empty((rows.shape[0], self.hidden_size), dtype=torch.float32, device=x.device)
        for e, (gate_up, fused, down) in enumerate(self.per_expert):
            lo, hi = bounds[e], bounds[e + 1]
            if hi > lo:
                act = self._activation(ctx, gathered[lo:hi], gate_up, fused)
                y[lo:hi].copy_(linear(ctx, act, down, out_dtype=torch.float32))
        return ops.moe_combine(y, where, weights)

    def forward(self, ctx, x):
        x = ops.materialize(x)
        chosen, weights, dense = ops.moe_router(x, self.router, self.top, over_all=self.route == "softmax_renorm", scale=self.scale)
        if (self.per_expert and x.shape[0] >= self.GROUPED_FROM and not getattr(ctx, "all_decode", True)
                and not torch.cuda.is_current_stream_capturing()):
            out = self._grouped(ctx, x, chosen, weights)
            return out if self.float32_out else out.to(x.dtype)
        act = self._activation(ctx, x, self.w_gate_up, self.fused, dense)
        if self.float32_out:
            return linear(ctx, act, self.w_down, out_dtype=torch.float32)
        return linear(ctx, act, self.w_down, allow_partial=True)


register_part("feed_forward", "moe", ExpertMixture, replace=True)
