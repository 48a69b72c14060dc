"""Two mixers side by side: both read the same input, each keeps what it
needs in a cache entry of its own, and the result is
left_scale * left + right_scale * right (summed in float32)."""
from __future__ import annotations

import torch

from .. import ops
from ..config.spec import CacheNeed, PartSpec
from .registry import CacheView, Runtime, StepContext, WeightStore, build_part, graph_safe, register_part


class ParallelMixers:
    kind = "parallel_mixers"

    def __init__(self, spec: PartSpec, weights: WeightStore, runtime: Runtime):
        self.left = build_part("mixer", spec["left"], weights, runtime)
        self.right = build_part("mixer", spec["right"], weights, runtime)
        self.left_scale, self.right_scale = float(spec["left_scale"]), float(spec["right_scale"])
        self.graph_safe = graph_safe(self.left) and graph_safe(self.right)

    def parts(self):
        return [self.left, self.right]

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="several", members=(self.left.cache_need(), self.right.cache_need()))

    def forward_pair(self, x: torch.Tensor, ctx: StepContext, cache: CacheView):
        """(left result, right result, (left_scale, right_scale)) for a caller
        that adds them up itself in a pass it makes anyway."""
        if len(cache.members) != 2:
            raise ValueError("two mixers side by side need a cache view with two members")
        left = self.left.forward(x, ctx, cache.members[0])
        right = self.right.forward(x, ctx, cache.members[1])
        return left, right, (self.left_scale, self.right_scale)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        left, right, (a, b) = self.forward_pair(x, ctx, cache)
        return ops.weighted_sum(left, right, a, b)

    def weight_bytes(self) -> int:
        return self.left.weight_bytes() + self.right.weight_bytes()


register_part("mixer", "parallel_mixers", lambda spec, weights, runtime: ParallelMixers(spec, weights, runtime))
