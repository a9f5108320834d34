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

    def __init__(self, mixer, feed_forward, norms, *, prefix: str = "", hidden_size: int = 0, residual_mult: float = 1.0, unused_names=()):
        """``residual_mult``: a constant that every sublayer's output is multiplied by before it is added, ``x + m *
        sublayer(norm(x))`` (1: the plain sum).  A layer may have no feed-forward (``prenorm_mixer_only``).
        ``unused_names``: tensors of the layer that a checkpoint may carry although the layer has no use for them."""
        super().__init__(mixer, feed_forward, norms)
        self.residual_mult, self.hidden = float(residual_mult), hidden_size
        self.mult: torch.Tensor | None = None
        self.unused = [prefix + name for name in unused_names]

    def weight_specs(self) -> list[WeightSpec]:
        return super().weight_specs() + [WeightSpec(name, (), role="vector", optional=True) for name in self.unused]

    def load(self, tensors) -> None:
        super().load(tensors)
        if self.residual_mult != 1.0:  # the norm that adds a pending output takes a factor per column
            self.mult = torch.full((self.hidden,), self.residual_mult, dtype=torch.float32, device=self.mixer_norm.weight.device)

    def forward(self, state: Residual, ctx: StepContext, cache: LayerCache) -> None:
        h = self.mixer_norm.forward(state, ctx, ctx.dtype)
        state.add(self.mixer.forward(h, ctx, cache), self.mult)
        if self.feed_forward is not None:
            h = self.feed_forward_norm.forward(state, ctx, ctx.dtype)
            state.add(self.feed_forward.forward(h, ctx), self.mult)


@register("block", "prenorm_mixer_only")
class PreNormMixerOnlyBlock(PreNormBlock):
    """The same arrangement for a layer without a feed-forward: one norm."""

    NORMS = ("mixer",)


@register("block", "hyper_prenorm")
class HyperConnectionBlock(Block):
    """Pre-norm sublayers on several residual streams ``x_1 .. x_N`` (hyper-connections) in the place of one.  Sublayer
    ``q`` (the mixer, then the feed-forward) has learned ``read_q [N]``, ``mix_q [N, N]`` (indexed ``[from, to]``) and
    ``share_q [N]``::

        u = sum_s read_q[s] x_s        y = sublayer_q(norm_q(u))        x_t <- sum_s mix_q[s, t] x_s + m * share_q[t] * y

    with all streams updated at once from the old ones and ``m`` a constant of the model (``residual_mult``).  At the
    model's start every stream is the embedding's output; at its end the residual is the sum of the streams (the
    final norm reads it with ``Residual.stream_read = None``).  The update that a sublayer's output is owed happens
    inside the kernel of the norm that follows, together with that norm's read, in 32-bit."""

    capturable = True

    def __init__(self, mixer, feed_forward, norms, *, prefix: str, hidden_size: int, streams: int, names, residual_mult: float = 1.0, unused_names=()):
        """``names``: for ``"mixer"`` (and ``"feed_forward"``) the tensor names of ``read``, ``mix`` and ``share``
        behind the layer's prefix.  ``unused_names``: tensors of the layer that a checkpoint may carry although the
        layer has no use for them (the norm and the coefficients of a feed-forward that the layer does not have)."""
        super().__init__(mixer, feed_forward, norms)
        if not 1 <= streams <= 8:
            raise ValueError(f"hyper_prenorm takes 1 to 8 residual streams, got {streams}")
        wanted = {"mixer"} if feed_forward is None else {"mixer", "feed_forward"}
        if set(names) != wanted or any(set(group) != {"read", "mix", "share"} for group in names.values()):
            raise ValueError(f"hyper_prenorm wants the names of read, mix and share for {sorted(wanted)}")
        self.count, self.hidden, self.mult = int(streams), hidden_size, float(residual_mult)
        self.names = {sub: {key: prefix + name for key, name in group.items()} for sub, group in names.items()}
        self.coefficients: dict[str, dict[str, torch.Tensor]] = {}
        self.unused = [prefix + name for name in unused_names]

    def weight_specs(self) -> list[WeightSpec]:
        specs = super().weight_specs()
        for group in self.names.values():  # the streams are 32-bit, and so is what multiplies them
            specs += [
                WeightSpec(group["read"], (self.count,), role="vector", init="ones_normal"),
                WeightSpec(group["share"], (self.count,), role="vector", init="ones_normal"),
                WeightSpec(group["mix"], (self.count, self.count), role="vector", init="eye_normal"),
            ]
        return specs + [WeightSpec(name, (), role="vector", optional=True) for name in self.unused]

    def load(self, tensors) -> None:
        super().load(tensors)
        self.coefficients = {sub: {key: tensors[name] for key, name in group.items()} for sub, group in self.names.items()}

    def _sublayer(self, which: str, norm, state: Residual, ctx: StepContext, run) -> None:
        if state.streams is None:  # the model's first sublayer: the streams all equal the embedding's output
            flat = ctx.buffer("residual.streams", (ctx.num_tokens, self.count * self.hidden), torch.float32)
            state.streams = flat.view(self.count, ctx.num_tokens, self.hidden)  # stream after stream
            state.streams_unwritten = True
        elif state.streams.shape[0] != self.count:
            raise ValueError("every layer of a model has the same number of residual streams")
        held = self.coefficients[which]
        state.stream_read = held["read"]
        h = norm.forward(state, ctx, ctx.dtype)
        state.add(run(h))
        state.stream_update = (held["mix"], held["share"], self.mult)

    def forward(self, state: Residual, ctx: StepContext, cache: LayerCache) -> None:
        self._sublayer("mixer", self.mixer_norm, state, ctx, lambda h: self.mixer.forward(h, ctx, cache))
        if self.feed_forward is not None:
            self._sublayer("feed_forward", self.feed_forward_norm, state, ctx, lambda h: self.feed_forward.forward(h, ctx))


@register("block", "hyper_prenorm_mixer_only")
class HyperConnectionMixerOnlyBlock(HyperConnectionBlock):
    """The same arrangement for a layer without a feed-forward: one norm."""

    NORMS = ("mixer",)


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
