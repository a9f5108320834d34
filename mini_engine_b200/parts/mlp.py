"""Dense gated feed-forward (SwiGLU) as a part.

``y = (silu(x Wg^T) * (x Wu^T)) Wd^T`` with ``silu(a) = a * sigmoid(a)`` and no biases
(src/mini_engine/model.py:122-131 of YuvGev00/mini-engine).  Gate and up run as one product
on the row-concatenated weight; on the tensor-core path the activation is applied in that
product's epilogue, so the ``[T, 2 * inter]`` intermediate never reaches memory.

The gate has three constants for models whose gated unit differs: ``y = g * sigmoid(gate_slope * g) *
(u + up_offset)`` with ``g = min(x Wg^T, limit)`` and ``u = clamp(x Wu^T, -limit, limit)`` when a
``limit`` is given.  Slope 1, no limit and offset 0 are SwiGLU.  ``activation="gelu_tanh"`` gates with
``0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3)))`` in the place of ``g * sigmoid(gate_slope * g)``.

``mlp`` is the feed-forward without a gate, ``y = act(x Wu^T) Wd^T`` with ``act`` the square of relu (``relu_squared``),
``relu``, ``silu`` or ``gelu_tanh``: the up product's partial sums meet in the activation kernel, which rounds once.
"""

from __future__ import annotations

from typing import Mapping

import torch

from mini_engine_b200.csrc import ops
from mini_engine_b200.parts.base import FeedForward, StepContext, register
from mini_engine_b200.parts.linear import GatedLinear, Linear
from mini_engine_b200.weights.loader import WeightSpec


@register("feed_forward", "gated_mlp")
class GatedMLP(FeedForward):
    capturable = True

    def __init__(
        self,
        prefix: str,
        hidden_size: int,
        *,
        intermediate_size: int,
        activation: str = "silu",
        names: Mapping[str, str] | None = None,
        gate_slope: float = 1.0,
        limit: float | None = None,
        up_offset: float = 0.0,
    ):
        if activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"gated_mlp gates with 'silu' or 'gelu_tanh', got {activation!r}")
        self.activation = activation
        if limit is not None and not limit > 0:
            raise ValueError(f"the limit of the gated unit must be positive, got {limit}")
        self.hidden, self.inter = hidden_size, intermediate_size
        self.gate_slope, self.limit, self.up_offset = float(gate_slope), limit, float(up_offset)
        defaults = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}
        self.names = {key: prefix + (names or {}).get(key, value) for key, value in defaults.items()}
        self.gate_up: GatedLinear | None = None
        self.down: Linear | None = None

    def weight_specs(self) -> list[WeightSpec]:
        n = self.names
        return [
            WeightSpec(n["gate"], (self.inter, self.hidden)),
            WeightSpec(n["up"], (self.inter, self.hidden)),
            WeightSpec(n["down"], (self.hidden, self.inter)),
        ]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        self.gate_up = GatedLinear(
            torch.cat((tensors[n["gate"]], tensors[n["up"]]), dim=0).contiguous(),
            slope=self.gate_slope, limit=self.limit, offset=self.up_offset, activation=self.activation,
        )  # fmt: skip
        self.down = Linear(tensors[n["down"]])

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        act = self.gate_up.forward(h, ctx, "mlp")
        return self.down.forward(act, ctx, "mlp.down")


@register("feed_forward", "mlp")
class PlainMLP(FeedForward):
    capturable = True

    def __init__(
        self, prefix: str, hidden_size: int, *, intermediate_size: int, activation: str = "relu_squared",
        names: Mapping[str, str] | None = None,
    ):  # fmt: skip
        if activation not in ops.PLAIN_ACTIVATIONS:
            raise ValueError(f"mlp: activation must be one of {sorted(ops.PLAIN_ACTIVATIONS)}, got {activation!r}")
        if intermediate_size < 1:
            raise ValueError("mlp: the intermediate size must be positive")
        self.hidden, self.inter, self.activation = hidden_size, intermediate_size, activation
        defaults = {"up": "up_proj.weight", "down": "down_proj.weight"}
        self.names = {key: prefix + (names or {}).get(key, value) for key, value in defaults.items()}
        self.up: Linear | None = None
        self.down: Linear | None = None

    def weight_specs(self) -> list[WeightSpec]:
        return [
            WeightSpec(self.names["up"], (self.inter, self.hidden)),
            WeightSpec(self.names["down"], (self.hidden, self.inter)),
        ]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.up, self.down = Linear(tensors[self.names["up"]]), Linear(tensors[self.names["down"]])

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        sums = self.up.forward(h, ctx, "mlp.up")
        act = ctx.buffer("mlp.plain_act", (h.shape[0], self.inter), h.dtype)
        ops.activation(sums, act, self.activation)
        return self.down.forward(act, ctx, "mlp.plain_down")
