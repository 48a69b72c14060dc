"""Arrangement of one layer's parts.

``prenorm_residual`` is the reference's layer
(crates/models/qwen/src/forward.rs:1856-1885, :1889-1922):
r = x + mixer(norm1(x)); x' = r + feed_forward(norm2(r)). The residual stream
is float32; a block receives the previous block's output not yet added
(``pending``) so that every residual sum runs inside the norm kernel that
follows it.

``sandwich_residual`` puts a second norm behind each sublayer:
r = x + post1(mixer(norm1(x))); x' = r + post2(feed_forward(norm2(r))), the
feed-forward half being optional. What a sublayer leaves is handed on with
the norm it still has to pass (``Pending``), so that this norm, the residual
sum and the next sublayer's norm run as one kernel.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..config.spec import LayerSpec
from .registry import CacheView, Pending, Runtime, StepContext, WeightStore, build_part, register_part


class PreNormResidualBlock:
    kind = "prenorm_residual"

    def __init__(self, layer: LayerSpec, weights: WeightStore, runtime: Runtime):
        self.name = layer.name
        self.mixer_norm = build_part("norm", layer.mixer_norm, weights, runtime)
        self.mixer = build_part("mixer", layer.mixer, weights, runtime)
        self.feed_forward_norm = build_part("norm", layer.feed_forward_norm, weights, runtime)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, weights, runtime)
        self.dtype = runtime.dtype
        # A mixer may leave its output as summands [parts, tokens, hidden] when
        # the norm that takes it next adds them up in its own pass over the row.
        summands = getattr(self.mixer, "forward_summands", None)
        self.mix = summands if summands is not None and getattr(self.feed_forward_norm, "adds_summands", False) \
            else self.mixer.forward

    def parts(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def forward(self, residual: torch.Tensor, pending, ctx: StepContext,
                cache: CacheView) -> torch.Tensor:
        """``residual`` (float32, updated in place) plus ``pending`` (a tensor,
        or a ``Pending`` that carries the norm it passes first) is the layer's
        input; returns the feed-forward output, to be added by whoever runs
        next."""
        mixer_in = self.mixer_norm.add_forward(residual, pending, self.dtype)
        mixed = self.mix(mixer_in, ctx, cache)
        feed_in = self.feed_forward_norm.add_forward(residual, mixed, self.dtype)
        return self.feed_forward.forward(feed_in, ctx)


class SandwichNormBlock:
    kind = "sandwich_residual"

    def __init__(self, layer: LayerSpec, weights: WeightStore, runtime: Runtime):
        self.name = layer.name
        if layer.mixer_post_norm is None:
            raise ValueError(f"{layer.name}: a sandwich block needs the norm behind its mixer")
        self.mixer_norm = build_part("norm", layer.mixer_norm, weights, runtime)
        self.mixer = build_part("mixer", layer.mixer, weights, runtime)
        self.mixer_post_norm = build_part("norm", layer.mixer_post_norm, weights, runtime)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, weights, runtime)
        self.feed_forward_norm = self.feed_forward_post_norm = None
        if self.feed_forward is not None:
            if layer.feed_forward_norm is None or layer.feed_forward_post_norm is None:
                raise ValueError(f"{layer.name}: a feed-forward in a sandwich block needs both of its norms")
            self.feed_forward_norm = build_part("norm", layer.feed_forward_norm, weights, runtime)
            self.feed_forward_post_norm = build_part("norm", layer.feed_forward_post_norm, weights, runtime)
        self.dtype = runtime.dtype
        # Summands [parts, tokens, hidden] are taken where the kernel that adds
        # the mixer's output up is known to be this block's own.
        summands = getattr(self.mixer, "forward_summands", None)
        fused = (self.feed_forward is not None and getattr(self.feed_forward_norm, "adds_summands", False)
                 and getattr(self.mixer_post_norm, "adds_summands", False))
        self.mix = summands if summands is not None and fused else self.mixer.forward

    def parts(self):
        return [self.mixer_norm, self.mixer, self.mixer_post_norm, self.feed_forward_norm, self.feed_forward,
                self.feed_forward_post_norm]

    def forward(self, residual: torch.Tensor, pending, ctx: StepContext, cache: CacheView):
        mixer_in = self.mixer_norm.add_forward(residual, pending, self.dtype)
        mixed = Pending(self.mix(mixer_in, ctx, cache), self.mixer_post_norm)
        if self.feed_forward is None:
            return mixed
        feed_in = self.feed_forward_norm.add_forward(residual, mixed, self.dtype)
        return Pending(self.feed_forward.forward(feed_in, ctx), self.feed_forward_post_norm)


register_part("block", "sandwich_residual",
              lambda layer, weights, runtime: SandwichNormBlock(layer, weights, runtime))
register_part("block", "prenorm_residual",
              lambda layer, weights, runtime: PreNormResidualBlock(layer, weights, runtime))
