"""A feed-forward made of many small gated units ("experts") of which every token uses a few.

Router: ``s = sigmoid(W_r h)`` in 32-bit.  The units form ``group_count`` equal groups of neighbours; a group is
valued by the sum of its two largest scores and only units of the ``group_keep`` best groups are eligible; the
``top`` eligible units with the largest scores are chosen, with weights ``s / (sum of the chosen s + 1e-20) *
weight_scale``.  Unit ``e``: ``g = min(W_gate h, limit)``, ``u = clamp(W_up h, -limit, limit)``, ``W_down (g *
sigmoid(gate_slope * g) * (u + up_offset))`` (the constants of :mod:`~mini_engine_b200.parts.mlp`).  The output is
the weighted sum of the chosen units' outputs.

Options: ``router_bias`` adds a learned number per unit to ``W_r h``; ``scoring="softmax_chosen"`` chooses the ``top``
units with the largest logits and weighs them by the softmax over the chosen logits only; ``shared_intermediate_size``
adds a gated unit of that width (tensors ``shared``) that runs for every token, its output added with weight one.

How it runs, two forms; neither has a shape that depends on the choice, so both can be captured in a graph, and in
both a token's result does not depend on the rest of the batch.

* *All units, masked* (few tokens, float32, sizes that the tensor-core product does not take): all units' gate and
  up matrices are one row-concatenated weight and all down matrices one column-concatenated weight.  The routing
  kernel leaves a dense map ``[T, units]`` of weights (zero for units that a token did not choose); the activation
  kernel multiplies every unit's features by its weight for the token; the down product then *is* the weighted sum
  over the chosen units.  A step of few tokens reads nearly all units' weights anyway.
* *Rows sorted by unit* (bfloat16 steps of ``SORTED_MIN_TOKENS`` tokens and more, and steps of so few tokens that
  their choices cannot touch half of the units): every (token, choice) gets a row
  in an array sorted by unit, each unit's run padded to whole tiles of 128 rows; the tokens' inputs are gathered
  into it; a grouped tensor-core product whose tiles read the weights of their run's unit forms the gated
  activations (the gate in its epilogue), a second one the down products, and a last kernel adds a token's rows
  with their weights in the order of its choices.  Only chosen units are computed.
"""

from __future__ import annotations

from typing import Mapping

import torch

from mini_engine_b200.csrc import ops
from mini_engine_b200.parts.base import FeedForward, StepContext, register
from mini_engine_b200.parts.linear import GatedLinear, Linear
from mini_engine_b200.weights.loader import WeightSpec

# From this many tokens on a bfloat16 step sorts its rows by unit and computes only chosen units.  Below, the
# masked form's two products over all units cost less than the sorted form's five launches and padded tiles.
SORTED_MIN_TOKENS = 256


@register("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    capturable = True

    def __init__(
        self,
        prefix: str,
        hidden_size: int,
        *,
        units: int,
        top: int,
        intermediate_size: int,
        group_count: int = 1,
        group_keep: int = 1,
        weight_scale: float = 1.0,
        gate_slope: float = 1.0,
        limit: float | None = None,
        up_offset: float = 0.0,
        names: Mapping[str, str] | None = None,
        router_bias: bool = False,
        scoring: str = "sigmoid",
        shared_intermediate_size: int | None = None,
    ):
        if scoring not in ops.ROUTE_SCORINGS:
            raise ValueError(f"routed_experts: scoring must be one of {sorted(ops.ROUTE_SCORINGS)}, got {scoring!r}")
        self.router_bias, self.scoring = bool(router_bias), scoring
        self.shared_inter = int(shared_intermediate_size or 0)
        if self.shared_inter < 0:
            raise ValueError("routed_experts: the shared unit's width must be positive")
        if min(units, top, intermediate_size, group_count, group_keep) < 1:
            raise ValueError("routed_experts: sizes must be positive")
        if units % group_count or group_keep > group_count or top > group_keep * (units // group_count):
            raise ValueError(
                f"routed_experts: {units} units do not form {group_count} equal groups of which {group_keep} hold {top} choices"
            )
        if limit is not None and not limit > 0:
            raise ValueError(f"the limit of the gated unit must be positive, got {limit}")
        self.hidden, self.units, self.top, self.inter = hidden_size, units, top, intermediate_size
        self.group_count, self.group_keep, self.weight_scale = group_count, group_keep, float(weight_scale)
        self.gate_slope, self.limit, self.up_offset = float(gate_slope), limit, float(up_offset)
        defaults = {"router": "router.weight", "unit": "experts.{index}.", "gate": "gate_proj.weight",
                    "up": "up_proj.weight", "down": "down_proj.weight", "router_bias": "router.bias",
                    "shared": "shared_expert."}  # fmt: skip
        self.names = {key: (names or {}).get(key, value) for key, value in defaults.items()}
        self.prefix = prefix
        self.gate_up: Linear | None = None
        self.down: Linear | None = None
        self.router: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None
        self.shared_gate_up: GatedLinear | None = None
        self.shared_down: Linear | None = None
        self.sorted_gate_up = self.sorted_down = None  # plans of the grouped products, when the sizes allow them

    def _name(self, unit: int, which: str) -> str:
        return self.prefix + self.names["unit"].format(index=unit) + self.names[which]

    def weight_specs(self) -> list[WeightSpec]:
        specs = []
        for unit in range(self.units):
            specs += [
                WeightSpec(self._name(unit, "gate"), (self.inter, self.hidden)),
                WeightSpec(self._name(unit, "up"), (self.inter, self.hidden)),
                WeightSpec(self._name(unit, "down"), (self.hidden, self.inter)),
            ]
        # the router is applied in 32-bit
        specs.append(WeightSpec(self.prefix + self.names["router"], (self.units, self.hidden), role="vector", init="small_normal"))
        if self.router_bias:
            specs.append(WeightSpec(self.prefix + self.names["router_bias"], (self.units,), role="vector", init="small_normal"))
        if self.shared_inter:
            shared = self.prefix + self.names["shared"]
            specs += [
                WeightSpec(shared + self.names["gate"], (self.shared_inter, self.hidden)),
                WeightSpec(shared + self.names["up"], (self.shared_inter, self.hidden)),
                WeightSpec(shared + self.names["down"], (self.hidden, self.shared_inter)),
            ]
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        gates = [tensors[self._name(unit, "gate")] for unit in range(self.units)]
        ups = [tensors[self._name(unit, "up")] for unit in range(self.units)]
        self.gate_up = Linear(torch.cat(gates + ups, dim=0).contiguous())  # [all gates | all ups]
        self.down = Linear(torch.cat([tensors[self._name(unit, "down")] for unit in range(self.units)], dim=1).contiguous())
        self.router = tensors[self.prefix + self.names["router"]]
        if self.router_bias:
            self.bias = tensors[self.prefix + self.names["router_bias"]]
        if self.shared_inter:
            shared = self.prefix + self.names["shared"]
            self.shared_gate_up = GatedLinear(
                torch.cat((tensors[shared + self.names["gate"]], tensors[shared + self.names["up"]]), dim=0).contiguous(),
                slope=self.gate_slope, limit=self.limit, offset=self.up_offset,
            )  # fmt: skip
            self.shared_down = Linear(tensors[shared + self.names["down"]])
        if gates[0].dtype == torch.bfloat16 and ops.tensor_core_gemm_supports(self.inter, self.hidden) and ops.tensor_core_gemm_supports(self.hidden, self.inter):
            # unit after unit: [gate rows; up rows] of each, and the down matrices stacked by rows
            stacked = torch.cat([torch.cat((gate, up), dim=0) for gate, up in zip(gates, ups)], dim=0).contiguous()
            self.sorted_gate_up = ops.GemmPlan(stacked)
            self.sorted_down = ops.GemmPlan(torch.cat([tensors[self._name(unit, "down")] for unit in range(self.units)], dim=0).contiguous())

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        tokens = h.shape[0]
        weights = ctx.buffer("routed.weights", (tokens, self.units), torch.float32)
        chosen = ctx.buffer("routed.chosen", (tokens, self.top), torch.int32)
        chosen_weight = ctx.buffer("routed.chosen_weight", (tokens, self.top), torch.float32)
        ops.route(
            h=h, router=self.router, weights=weights, chosen=chosen, chosen_weight=chosen_weight, top=self.top,
            group_count=self.group_count, group_keep=self.group_keep, weight_scale=self.weight_scale, bias=self.bias,
            scoring=self.scoring,
        )  # fmt: skip
        routed = self._forward_routed(h, ctx, chosen, chosen_weight, weights)
        if not self.shared_inter:
            return routed
        act = self.shared_gate_up.forward(h, ctx, "routed.shared")
        shared = self.shared_down.forward(act, ctx, "routed.shared_down")
        out = ctx.buffer("routed.sum", (tokens, self.hidden), torch.float32)
        ops.branch_sum([(routed, 1.0), (shared, 1.0)], out)  # each output whole before the two meet
        return out.unsqueeze(0)

    def _forward_routed(self, h: torch.Tensor, ctx: StepContext, chosen, chosen_weight, weights) -> torch.Tensor:
        tokens = h.shape[0]
        # Many tokens: only chosen units are computed.  Very few: only chosen units' weights are read.  The choice
        # depends on the token count alone, so a captured step always takes the form it was captured with.
        if self.sorted_gate_up is not None and (tokens >= SORTED_MIN_TOKENS or 2 * tokens * self.top <= self.units):
            return self._forward_sorted(h, ctx, chosen, chosen_weight)
        both = self.gate_up.forward(h, ctx, "routed.gate_up")
        act = ctx.buffer("routed.act", (tokens, self.units * self.inter), ctx.dtype)
        ops.swiglu(both, act, self.gate_slope, self.limit, self.up_offset, group_weight=weights)
        return self.down.forward(act, ctx, "routed.down")

    def _forward_sorted(self, h: torch.Tensor, ctx: StepContext, chosen: torch.Tensor, chosen_weight: torch.Tensor) -> torch.Tensor:
        tokens, pad = h.shape[0], ops.GROUP_PAD
        # every unit's run may end in a partly filled tile; the capacity is a function of the step's token count alone
        capacity = -(-(tokens * self.top + self.units * (pad - 1)) // pad) * pad
        grow = ctx.workspace.growing
        row_of = grow("routed.row_of", (tokens, self.top), torch.int32)
        token_of = grow("routed.token_of", (capacity,), torch.int32)
        unit_of_block = grow("routed.unit_of_block", (capacity // pad,), torch.int32)
        ops.sort_by_unit(chosen=chosen, units=self.units, pad=pad, row_of=row_of, token_of=token_of, unit_of_block=unit_of_block)
        rows = grow("routed.rows", (capacity, self.hidden), h.dtype)
        ops.gather_rows(h, token_of, rows)
        act = grow("routed.sorted_act", (capacity, self.inter), h.dtype)
        ops.gemm_tensor_core_grouped(
            self.sorted_gate_up, rows, act, unit_of_block, 2 * self.inter, self.inter, dual_rows=self.inter,
            slope=self.gate_slope, limit=self.limit, offset=self.up_offset,
        )  # fmt: skip
        down = grow("routed.sorted_down", (capacity, self.hidden), torch.float32)
        ops.gemm_tensor_core_grouped(self.sorted_down, act, down, unit_of_block, self.hidden, self.hidden)
        out = ctx.buffer("routed.out", (tokens, self.hidden), torch.float32)
        ops.combine_rows(down, row_of, chosen_weight, out)
        return out.unsqueeze(0)
