"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, the weight multiplying
directly (crates/models/qwen/src/forward.rs:2442-2449). Sum of squares and
scale are float32 in both precisions. A checkpoint may store the weight around
zero (``one_plus``): the factor is then 1 + w, formed once in float32 when the
part is built."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..config.spec import PartSpec
from .registry import Pending, Runtime, WeightStore, register_part


class RMSNorm:
    kind = "rmsnorm"
    adds_summands = True   # add_forward also takes [parts, rows, size]: a sum its producer left in parts

    def __init__(self, weight: torch.Tensor, eps: float, runtime: Runtime, one_plus: bool = False):
        weight = weight.to(device=runtime.device, dtype=torch.float32)
        self.weight = (weight + 1.0 if one_plus else weight).contiguous()
        self.size = self.weight.numel()
        self.eps = float(eps)

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype,
                rows_index: Optional[torch.Tensor] = None) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps, out_dtype, rows_index=rows_index)

    def add_forward(self, residual: torch.Tensor, delta, out_dtype: torch.dtype) -> torch.Tensor:
        """residual += delta (float32, in place), then the norm of the sum.
        ``delta`` may be float32 ``[parts, rows, size]``: its parts are added up
        first. A ``Pending`` delta passes its own norm before the sum, in the
        same pass over the row when that norm is an RMSNorm too."""
        if delta is None:
            return ops.rmsnorm(residual, self.weight, self.eps, out_dtype)
        if isinstance(delta, Pending):
            if isinstance(delta.norm, RMSNorm):
                return ops.postnorm_add_rmsnorm(residual, delta.delta, delta.norm.weight, delta.norm.eps,
                                                self.weight, self.eps, out_dtype)
            delta.norm.add_normed(residual, delta.delta)
            return ops.rmsnorm(residual, self.weight, self.eps, out_dtype)
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, out_dtype)

    def add_normed(self, residual: torch.Tensor, delta: torch.Tensor) -> None:
        """residual += norm(delta) (float32, in place): this norm as the one a
        sublayer's output passes on its way into the residual stream."""
        ops.postnorm_add_rmsnorm(residual, delta, self.weight, self.eps)


def _build(spec: PartSpec, weights: WeightStore, runtime: Runtime) -> RMSNorm:
    weight = weights.take(spec["weight"])
    if weight.numel() != spec["size"]:
        raise ValueError(f"{spec['weight']} has {weight.numel()} values, the norm is over {spec['size']}")
    return RMSNorm(weight, spec["eps"], runtime, one_plus=bool(spec.get("one_plus", False)))


register_part("norm", "rmsnorm", _build)
