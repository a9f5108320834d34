"""Arrangements of a layer's parts around the residual stream."""

from __future__ import annotations

import torch

from mini_engine_b200.csrc import ops
from mini_engine_b200.parts.base import Block, LayerCache, Residual, StepContext, register
from mini_engine_b200.weights.loader import WeightSpec


@register("block", "prenorm")
class PreNormBlock(Block):
    """``h = x + mixer(norm(x))``, ``y = h + feed_forward(norm(h))``
    (src/mini_engine/model.py:149-150 of YuvGev00/mini-engine).  The two sums happen inside
    the norms that follow them (the last one inside the next layer's first norm or the
    model's final norm), in 32-bit."""

    capturable = True

    def forward(self, state: Residual, ctx: StepContext, cache: LayerCache) -> None:
        h = self.mixer_norm.forward(state, ctx, ctx.dtype)
        state.add(self.mixer.forward(h, ctx, cache))
        h = self.feed_forward_norm.forward(state, ctx, ctx.dtype)
        state.add(self.feed_forward.forward(h, ctx))


class _LayerScales:
    """Per-channel multipliers of a part's output ("layer scale"), one vector per part."""

    def __init__(self, prefix: str, hidden_size: int, names):
        self.hidden = hidden_size
        self.scale_names = {key: prefix + name for key, name in names.items()}
        self.scales: dict[str, torch.Tensor] = {}

    def specs(self) -> list[WeightSpec]:
        return [WeightSpec(name, (self.hidden,), role="vector", init="ones_normal") for name in self.scale_names.values()]

    def load(self, tensors) -> None:
        self.scales = {key: tensors[name] for key, name in self.scale_names.items()}


@register("block", "prenorm_scaled")
class ScaledPreNormBlock(Block):
    """``h = x + s_m * mixer(norm(x))``, ``y = h + s_f * feed_forward(norm(h))`` with the per-channel
    vectors ``s_m``, ``s_f`` of the layer (a layer scale).  The products and the sums happen inside
    the norm that follows, in 32-bit: ``x + s * (sum of the part's partial sums)``."""

    capturable = True

    def __init__(self, mixer, feed_forward, norms, *, prefix: str, hidden_size: int, scale_names, unused_names=()):
        """``unused_names``: tensors of the layer that a checkpoint may carry although the layer has
        no use for them (the feed-forward's norm and scale of a layer without a feed-forward)."""
        super().__init__(mixer, feed_forward, norms)
        self.unused = [prefix + name for name in unused_names]
        wanted = {"mixer"} if feed_forward is None else {"mixer", "feed_forward"}
        if set(scale_names) != wanted:
            raise ValueError(f"the layer scales must be named for {sorted(wanted)}, got {sorted(scale_names)}")
        self.layer_scales = _LayerScales(prefix, hidden_size, scale_names)

    def weight_specs(self) -> list[WeightSpec]:
        unused = [WeightSpec(name, (), role="vector", optional=True) for name in self.unused]
        return super().weight_specs() + self.layer_scales.specs() + unused

    def load(self, tensors) -> None:
        super().load(tensors)
        self.layer_scales.load(tensors)

    def forward(self, state: Residual, ctx: StepContext, cache: LayerCache) -> None:
        h = self.mixer_norm.forward(state, ctx, ctx.dtype)
        state.add(self.mixer.forward(h, ctx, cache), self.layer_scales.scales["mixer"])
        if self.feed_forward is not None:
            h = self.feed_forward_norm.forward(state, ctx, ctx.dtype)
            state.add(self.feed_forward.forward(h, ctx), self.layer_scales.scales["feed_forward"])


@register("block", "prenorm_scaled_mixer_only")
class ScaledMixerOnlyBlock(ScaledPreNormBlock):
    """The same arrangement for a layer without a feed-forward: one norm, one layer scale."""

    NORMS = ("mixer",)


@register("block", "postnorm")
class PostNormBlock(Block):
    """The norm follows the sum: ``x = norm_m(alpha * x + mixer(x))``, then ``x = norm_f(alpha * x +
    feed_forward(x))``.  The sublayers read the stream itself (rounded to the compute dtype); each sum, in
    32-bit, and its norm are one kernel, which leaves the normalised row as the new stream."""

    capturable = True

    def __init__(self, mixer, feed_forward, norms, *, prefix: str, hidden_size: int, alpha: float = 1.0, unused_names=()):
        """``alpha``: what the stream is multiplied by before a sublayer's output is added.  ``unused_names``:
        tensors of the layer that a checkpoint may carry although the layer has no use for them."""
        super().__init__(mixer, feed_forward, norms)
        self.alpha = float(alpha)
        self.unused = [prefix + name for name in unused_names]

    def weight_specs(self) -> list[WeightSpec]:
        return super().weight_specs() + [WeightSpec(name, (), role="vector", optional=True) for name in self.unused]

    @staticmethod
    def _stream(state: Residual, ctx: StepContext) -> torch.Tensor:
        """The stream in the compute dtype."""
        if ctx.dtype == torch.float32:
            return state.x
        if state.rounded is None:
            state.rounded = ctx.buffer("block.rounded", tuple(state.x.shape), ctx.dtype)
            ops.round_rows(state.x, state.rounded)
        return state.rounded

    def forward(self, state: Residual, ctx: StepContext, cache: LayerCache) -> None:
        state.add(self.mixer.forward(self._stream(state, ctx), ctx, cache))
        self.mixer_norm.forward(state, ctx, ctx.dtype, residual_scale=self.alpha, keep_normed=True)
        if self.feed_forward is not None:
            state.add(self.feed_forward.forward(self._stream(state, ctx), ctx))
            self.feed_forward_norm.forward(state, ctx, ctx.dtype, residual_scale=self.alpha, keep_normed=True)


@register("block", "postnorm_mixer_only")
class PostNormMixerOnlyBlock(PostNormBlock):
    """The same arrangement for a layer without a feed-forward: one norm."""

    NORMS = ("mixer",)


@register("block", "parallel")
class ParallelBlock(Block):
    """One norm, both sublayers read its output: ``x = x + (mixer(norm(x)) + feed_forward(norm(x)))``.  The three
    terms (and the bias of the mixer's output projection) are added in 32-bit inside the next norm.  A layer may
    have no feed-forward."""

    capturable = True
    NORMS = ("mixer",)
    adds_output_bias = True

    def forward(self, state: Residual, ctx: StepContext, cache: LayerCache) -> None:
        h = self.mixer_norm.forward(state, ctx, ctx.dtype)
        state.add(self.mixer.forward(h, ctx, cache), bias=self.mixer.output_bias)
        if self.feed_forward is not None:
            state.add_beside(self.feed_forward.forward(h, ctx))
