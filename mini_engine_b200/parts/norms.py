"""RMSNorm and layer norm as parts.

``y = w * (x * rsqrt(mean(x^2) + eps))`` with the statistics in 32-bit, eps inside the root
(src/mini_engine/model.py:59-69 of YuvGev00/mini-engine).  The reference rounds the
normalised value to the model dtype before the weight multiply; here the whole expression
is evaluated in 32-bit and rounded once, which is at least as accurate.  The norm also
performs the residual sum that precedes it (see :class:`~mini_engine_b200.parts.base.Residual`).

``layernorm``: ``y = (x - mean(x)) / sqrt(var(x) + eps) * w + b`` with the variance as the mean of the
squared deviations, weight and bias of the layer, all in 32-bit.  Its residual sum also takes the bias of
an output projection and the output of a second sublayer that ran beside the first.
"""

from __future__ import annotations

from typing import Mapping

import torch

from mini_engine_b200.csrc import ops
from mini_engine_b200.parts.base import Norm, Residual, StepContext, register
from mini_engine_b200.weights.loader import WeightSpec


@register("norm", "rmsnorm")
class RMSNorm(Norm):
    capturable = True

    def __init__(
        self, prefix: str, hidden_size: int, *, name: str, eps: float, dim: int | None = None, offset: float = 0.0
    ):
        """``offset``: what is added to the stored weight before it multiplies (1 for a checkpoint that
        keeps its norm weights around zero: ``y = (1 + w) * x / rms(x)``); the sum is formed once, in 32-bit."""
        self.weight_name = prefix + name
        self.dim = dim or hidden_size
        self.eps = float(eps)
        self.offset = float(offset)
        self.weight: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        init = "ones_normal" if self.offset == 0.0 else "small_normal"
        return [WeightSpec(self.weight_name, (self.dim,), role="vector", init=init)]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name]
        if self.offset != 0.0:
            self.weight = (self.weight + self.offset).contiguous()

    def forward(
        self, state: Residual, ctx: StepContext, out_dtype, rows=None, residual_scale: float = 1.0, keep_normed: bool = False
    ) -> torch.Tensor:
        if state.pending_bias is not None or state.pending_more is not None:
            raise ValueError("rmsnorm adds one pending output without a bias")
        count = state.x.shape[0] if rows is None else rows.shape[0]
        out = ctx.buffer("norm.out" if rows is None else "norm.rows", (count, self.dim), out_dtype)
        if state.streams is not None:
            return self._forward_streams(state, out, rows, residual_scale, keep_normed)
        ops.add_rmsnorm(
            state.x, state.pending, self.weight, self.eps, out, rows, state.pending_scale, residual_scale, keep_normed
        )
        if rows is None:
            state.clear()
            state.rounded = out if keep_normed else None  # with keep_normed, `out` is the new stream, rounded
        return out


    def _forward_streams(self, state: Residual, out, rows, residual_scale, keep_normed) -> torch.Tensor:
        """Several residual streams: the pending output's update of all streams, their weighted sum and its norm are
        one kernel (see :class:`~mini_engine_b200.parts.base.Residual`)."""
        if residual_scale != 1.0 or keep_normed or state.pending_scale is not None:
            raise ValueError("rmsnorm over several residual streams stands in front of its sublayer: no factor, no scale, no write-back")
        if (state.pending is None) != (state.stream_update is None):
            raise RuntimeError("a pending output of a model with several streams comes with its update, and only with it")
        mix, share, mult = state.stream_update or (None, None, 1.0)
        ops.hyper_step(
            streams=state.streams, seed=state.x if state.streams_unwritten else None, pending=state.pending, mix=mix,
            share=share, mult=mult, read=state.stream_read, weight=self.weight, eps=self.eps, out=out, rows=rows,
        )  # fmt: skip
        if rows is None:
            if state.pending is not None:
                state.streams_unwritten = False
            state.clear()
            state.rounded = None
        return out


@register("norm", "layernorm")
class LayerNorm(Norm):
    capturable = True

    def __init__(self, prefix: str, hidden_size: int, *, name: str, eps: float, bias_name: str | None = None, dim: int | None = None):
        """``name``: the weight's tensor; ``bias_name``: the bias's (by default ``name + ".b"``)."""
        self.weight_name = prefix + name
        self.bias_name = prefix + (bias_name if bias_name is not None else name + ".b")
        self.dim = dim or hidden_size
        self.eps = float(eps)
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        return [
            WeightSpec(self.weight_name, (self.dim,), role="vector", init="ones_normal"),
            WeightSpec(self.bias_name, (self.dim,), role="vector", init="small_normal"),
        ]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight, self.bias = tensors[self.weight_name], tensors[self.bias_name]

    def forward(
        self, state: Residual, ctx: StepContext, out_dtype, rows=None, residual_scale: float = 1.0, keep_normed: bool = False
    ) -> torch.Tensor:
        if residual_scale != 1.0 or keep_normed or state.pending_scale is not None:
            raise ValueError("layernorm stands in front of its sublayers: no factor on the stream, no scale, no write-back")
        count = state.x.shape[0] if rows is None else rows.shape[0]
        out = ctx.buffer("norm.out" if rows is None else "norm.rows", (count, self.dim), out_dtype)
        ops.add_layernorm(
            state.x, state.pending, self.weight, self.bias, self.eps, out, rows, state.pending_more, state.pending_bias
        )
        if rows is None:
            state.clear()
            state.rounded = None
        return out
