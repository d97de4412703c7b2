"""Mixers side by side: every branch reads the same input; the result is the mean of the
branches' outputs, each first divided by its root mean square over the model width (`eps`)
and multiplied by a plain weight vector of its own (`<branch>.out`).

Parameter `branches` is a tuple of (name, PartSpec); any registered mixer may be a branch.
At most one branch may keep per-token entries in pages and at most one a state slot, since a
layer run has one paged cache and one state. The result is float32.

`merge` = "sum" with `scales` (one constant per branch) gives sum_b scales[b] * branch_b instead:
no norm, no weight vectors.
"""
from __future__ import annotations

from typing import Dict, Optional

from .. import ops
from ..config.schema import ConfigError, PartSpec
from ..weights.loader import WeightSpec
from .base import Mixer, PositionEncoding, part_factory, register_part


class BranchMixer(Mixer):
    def __init__(self, spec: PartSpec, hidden_size: int, position: Optional[PositionEncoding]):
        super().__init__(spec, hidden_size, position)
        self.merge = spec.get("merge", "unit_rms_mean")
        if self.merge not in ("unit_rms_mean", "sum"):
            raise ConfigError("branches: merge is 'unit_rms_mean' or 'sum'")
        self.eps = float(spec["eps"]) if self.merge == "unit_rms_mean" else 0.0
        self.scales = tuple(float(c) for c in (spec.get("scales") or ()))
        self.branches = []
        for name, branch_spec in spec["branches"]:
            self.branches.append((name, part_factory("mixer", branch_spec.kind)(branch_spec, hidden_size, None)))
        if not 1 <= len(self.branches) <= 4:
            raise ConfigError("branches: one to four branches are taken")
        if self.merge == "sum" and len(self.scales) != len(self.branches):
            raise ConfigError("branches: the sum needs one constant per branch")
        if sum(b.cache_spec() is not None for _, b in self.branches) > 1 or \
                sum(b.state_spec() is not None for _, b in self.branches) > 1:
            raise ConfigError("branches: at most one branch may keep pages and at most one a state slot")
        self.capture_safe = all(getattr(b, "capture_safe", True) for _, b in self.branches)
        self.out_weights = []

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {}
        for name, branch in self.branches:
            specs.update({f"{name}.{key}": w for key, w in branch.weight_specs().items()})
            if self.merge == "unit_rms_mean":
                specs[f"{name}.out"] = WeightSpec((self.hidden_size,), init="norm", std=0.1)
        return specs

    def load(self, tensors, dtype):
        self.out_weights = []
        for name, branch in self.branches:
            prefix = name + "."
            own = {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}
            if self.merge == "unit_rms_mean":
                self.out_weights.append(own.pop("out"))
            branch.load(own, dtype)
        if len({w.dtype for w in self.out_weights}) > 1:
            self.out_weights = [w.float() for w in self.out_weights]

    def setup(self, device, dtype):
        for _, branch in self.branches:
            branch.setup(device, dtype)

    def first_weight(self):
        return self.branches[0][1].first_weight()

    def cache_spec(self):
        return next((b.cache_spec() for _, b in self.branches if b.cache_spec() is not None), None)

    def state_spec(self):
        return next((b.state_spec() for _, b in self.branches if b.state_spec() is not None), None)

    def forward(self, ctx, x, cache, writes_cache: bool = True):
        outs = [branch.forward(ctx, x, cache, writes_cache) for _, branch in self.branches]
        if self.merge == "sum":
            return ops.branch_sum(outs, self.scales)
        return ops.branch_merge(outs, self.out_weights, self.eps)


register_part("mixer", "branches", BranchMixer, replace=True)
