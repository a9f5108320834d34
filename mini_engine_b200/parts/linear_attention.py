"""Gated linear attention as a mixer part: a matrix state per head instead of cached keys.

Per head, with ``q_t = (W_q h_t) * dim^-1/2``, ``k_t = W_k h_t`` (``dim`` channels) and ``v_t = W_v h_t``
(``vdim`` channels)::

    S_t = diag(alpha_t) S_(t-1) + k_t v_t^T        o_t = S_t^T q_t
    alpha_t = sigmoid(z_t)^(1/tau)                 z_t = W_a2 (W_a1 h_t) + b   (one decay per key channel)

Each head's ``o_t`` is divided by its root mean square over ``vdim`` and multiplied by a weight
``[vdim]`` shared by the heads; the heads are concatenated, multiplied by ``silu(W_g h_t)`` and projected
by ``W_o``.  The state ``[heads, dim, vdim]`` is float32, starts at zero and is carried from token to
token in the request's state slot of the cache manager; the decay (sigmoid, its logarithm, the power),
the recurrence and the unit norm are computed in 32-bit from the 32-bit sums of the projections.

The five projections of the input run as one product on the row-concatenated weight; the second,
small factor of the decay's low-rank projection is applied by the kernel that prepares q, k and the
decays of all tokens for the scan.

``retention`` is the same recurrence with a fixed decay per head in the place of the data-dependent one, ``S_t = a_h
S_(t-1) + k_t v_t^T``: q and k are rotated by position (rotate-half, on their first ``rotary_dim`` elements), k is
multiplied by ``dim^-1/2`` after its rotation, there are no biases and no decay projection; each head's ``o_t`` is divided
by its root mean square (no weight), multiplied by ``silu(W_g h_t)`` and projected.  It shares the scan and the finishing
kernel with the gated form; a kernel of its own rotates, scales and lays q, k and the decays out for the scan.  Portions
of more than ``CHUNKED_MIN_TOKENS`` tokens do not walk token by token: a constant decay gives the recurrence over a chunk
of 64 tokens a closed form (the state in front of the chunk, decayed, plus a causal product inside the chunk), which
three kernels compute with all chunks side by side, in float32.
"""

from __future__ import annotations

from typing import Mapping, Sequence

import torch

from mini_engine_b200.csrc import ops
from mini_engine_b200.config.model_spec import PartSpec
from mini_engine_b200.parts.base import LayerCache, Mixer, StateSpec, StepContext, build_part, register
from mini_engine_b200.parts.linear import Linear
from mini_engine_b200.weights.loader import WeightSpec


@register("mixer", "gated_linear_attention")
class GatedLinearAttention(Mixer):
    capturable = True
    # Prompt steps of a model with this mixer at widths of 4,096 stalled on a B200 when every kernel of the step
    # was launched as a programmatic dependent (after 5 to 12 steps of 2,048 tokens in a row) and ran through in
    # plain stream order; which kernels meet badly is not known, so such a model's steps run in order.
    programmatic_launch = False

    def __init__(
        self,
        prefix: str,
        hidden_size: int,
        *,
        num_heads: int,
        head_dim: int,
        value_dim: int,
        decay_rank: int,
        tau: float,
        norm_eps: float,
        query_scale: float | None = None,
        names: Mapping[str, str] | None = None,
    ):
        if min(num_heads, head_dim, value_dim, decay_rank) < 1 or not tau > 0:
            raise ValueError("gated_linear_attention: sizes and tau must be positive")
        self.hidden, self.heads, self.dim, self.vdim = hidden_size, num_heads, head_dim, value_dim
        self.rank, self.tau, self.eps = decay_rank, float(tau), float(norm_eps)
        self.q_scale = float(query_scale) if query_scale is not None else head_dim**-0.5
        defaults = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "g": "g_proj.weight",
                    "o": "o_proj.weight", "norm": "norm.weight", "a1": "decay_down.weight",
                    "a2": "decay_up.weight", "a2_bias": "decay_up.bias"}  # fmt: skip
        self.names = {key: prefix + (names or {}).get(key, value) for key, value in defaults.items()}
        # Columns of the fused input projection, in this order.
        widths = {"q": num_heads * head_dim, "k": num_heads * head_dim, "v": num_heads * value_dim,
                  "g": num_heads * value_dim, "a": decay_rank}  # fmt: skip
        self.columns, column = {}, 0
        for key, width in widths.items():
            self.columns[key] = column
            column += width
        self.proj: Linear | None = None
        self.out: Linear | None = None
        self.norm_weight = self.a2t = self.a2_bias = None

    def state(self) -> StateSpec:
        return StateSpec((self.heads, self.dim, self.vdim), torch.float32)

    def weight_specs(self) -> list[WeightSpec]:
        n, inner, outer = self.names, self.heads * self.dim, self.heads * self.vdim
        return [
            WeightSpec(n["q"], (inner, self.hidden)),
            WeightSpec(n["k"], (inner, self.hidden)),
            WeightSpec(n["v"], (outer, self.hidden)),
            WeightSpec(n["g"], (outer, self.hidden)),
            WeightSpec(n["o"], (self.hidden, outer)),
            WeightSpec(n["norm"], (self.vdim,), role="vector", init="ones_normal"),
            WeightSpec(n["a1"], (self.rank, self.hidden)),
            # the second factor of the decay enters the recurrence: kept and applied in 32-bit
            WeightSpec(n["a2"], (inner, self.rank), role="vector", init="small_normal"),
            WeightSpec(n["a2_bias"], (inner,), role="vector", init="ones_normal"),
        ]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        self.proj = Linear(torch.cat([tensors[n[key]] for key in ("q", "k", "v", "g", "a1")], dim=0).contiguous())
        self.out = Linear(tensors[n["o"]])
        self.norm_weight, self.a2_bias = tensors[n["norm"]], tensors[n["a2_bias"]]
        self.a2t = tensors[n["a2"]].t().contiguous()  # [rank, heads * dim]: the prepare kernel reads it along the channels

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        tokens = h.shape[0]
        proj = self.proj.forward(h, ctx, "gla.proj")
        raw = ctx.buffer("gla.raw", (tokens, self.heads * self.vdim), torch.float32)
        prepared = ctx.buffer("gla.prepared", (tokens, self.heads * 3 * self.dim), torch.float32)
        ops.gla_scan(
            proj=proj, columns=self.columns, a2t=self.a2t, a2_bias=self.a2_bias, ctx=ctx, state=cache.state, out=raw,
            prepared=prepared, q_scale=self.q_scale, tau=self.tau, heads=self.heads, dim=self.dim, vdim=self.vdim,
        )  # fmt: skip
        gated = ctx.buffer("gla.out", (tokens, self.heads * self.vdim), ctx.dtype)
        ops.gla_finish(
            o=raw, proj=proj, gate_column=self.columns["g"], weight=self.norm_weight, eps=self.eps, out=gated,
            heads=self.heads, vdim=self.vdim,
        )  # fmt: skip
        return self.out.forward(gated, ctx, "gla.o")


# An entry of at least this many tokens runs in chunks.  Below, the walk is as fast, and decoded tokens and short
# portions keep the bits of a token-by-token run.
CHUNKED_MIN_TOKENS = 33


@register("mixer", "retention")
class Retention(Mixer):
    capturable = True
    programmatic_launch = False  # it shares the scan kernel of the gated form, whose steps run in plain stream order

    def __init__(
        self,
        prefix: str,
        hidden_size: int,
        *,
        num_heads: int,
        head_dim: int,
        value_dim: int,
        decay: Sequence[float],
        norm_eps: float,
        position_encoding: PartSpec | None = None,
        key_scale: float | None = None,
        names: Mapping[str, str] | None = None,
    ):
        """``decay``: one constant per head, ``0 < a_h <= 1``; ``key_scale``: what rotated keys are multiplied by
        (default ``head_dim ** -0.5``); ``position_encoding``: a rotate-half rotation that the kernel applies, or none."""
        if min(num_heads, head_dim, value_dim) < 1:
            raise ValueError("retention: sizes must be positive")
        if head_dim > 192:
            raise ValueError(f"retention: the walking kernel keeps a state column of at most 192 key channels in registers, got {head_dim}")
        if len(decay) != num_heads or not all(0.0 < float(a) <= 1.0 for a in decay):
            raise ValueError(f"retention: one decay in (0, 1] per head ({num_heads}), got {list(decay)}")
        self.hidden, self.heads, self.dim, self.vdim = hidden_size, num_heads, head_dim, value_dim
        self.decay_values, self.eps = [float(a) for a in decay], float(norm_eps)
        self.k_scale = float(key_scale) if key_scale is not None else head_dim**-0.5
        self.position = None
        if position_encoding is not None:
            self.position = build_part("position_encoding", position_encoding, prefix, hidden_size)
        defaults = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "g": "g_proj.weight", "o": "o_proj.weight"}
        self.names = {key: prefix + (names or {}).get(key, value) for key, value in defaults.items()}
        widths = {"q": num_heads * head_dim, "k": num_heads * head_dim, "v": num_heads * value_dim, "g": num_heads * value_dim}
        self.columns, column = {}, 0
        for key, width in widths.items():  # columns of the fused input projection, in this order
            self.columns[key] = column
            column += width
        self.proj: Linear | None = None
        self.out: Linear | None = None
        self.decay: torch.Tensor | None = None
        self.chunked: bool | None = None  # whether the chunked kernels take the head sizes: asked once, on the device

    def state(self) -> StateSpec:
        return StateSpec((self.heads, self.dim, self.vdim), torch.float32)

    def weight_specs(self) -> list[WeightSpec]:
        n, inner, outer = self.names, self.heads * self.dim, self.heads * self.vdim
        specs = [
            WeightSpec(n["q"], (inner, self.hidden)),
            WeightSpec(n["k"], (inner, self.hidden)),
            WeightSpec(n["v"], (outer, self.hidden)),
            WeightSpec(n["g"], (outer, self.hidden)),
            WeightSpec(n["o"], (self.hidden, outer)),
        ]
        return specs + (self.position.weight_specs() if self.position is not None else [])

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        self.proj = Linear(torch.cat([tensors[n[key]] for key in ("q", "k", "v", "g")], dim=0).contiguous())
        self.out = Linear(tensors[n["o"]])
        # a decay enters the recurrence: the float32 nearest to the configuration's number, made from the double
        self.decay = torch.tensor(self.decay_values, dtype=torch.float64).to(torch.float32).to(tensors[n["q"]].device)
        if self.position is not None:
            self.position.load(tensors)

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        tokens = h.shape[0]
        table = self.position.step_angles(ctx) if self.position is not None else None
        if self.position is not None and table is None:
            raise ValueError("retention takes a rotation that its kernel applies, or none")
        proj = self.proj.forward(h, ctx, "retention.proj")
        raw = ctx.buffer("retention.raw", (tokens, self.heads * self.vdim), torch.float32)
        prepared = ctx.buffer("retention.prepared", (tokens, self.heads * 3 * self.dim), torch.float32)
        if self.chunked is None:
            self.chunked = ops.retention_chunked_supports(self.dim, self.vdim)
        chunk_min, chunk_state = 0, None
        if self.chunked and ctx.max_query_len >= CHUNKED_MIN_TOKENS:  # a step's longest entry is known on the host
            chunks = tokens // ops.RETENTION_CHUNK + ctx.num_entries
            chunk_min = CHUNKED_MIN_TOKENS
            chunk_state = ctx.workspace.growing("retention.chunks", (chunks, self.heads, self.dim, self.vdim), torch.float32)
        ops.retention_scan(
            proj=proj, columns=self.columns, cos_sin=table, decay=self.decay, k_scale=self.k_scale, ctx=ctx,
            state=cache.state, out=raw, prepared=prepared, heads=self.heads, dim=self.dim, vdim=self.vdim,
            chunk_min=chunk_min, chunk_state=chunk_state,
        )  # fmt: skip
        gated = ctx.buffer("retention.out", (tokens, self.heads * self.vdim), ctx.dtype)
        ops.gla_finish(
            o=raw, proj=proj, gate_column=self.columns["g"], weight=None, eps=self.eps, out=gated, heads=self.heads,
            vdim=self.vdim,
        )  # fmt: skip
        return self.out.forward(gated, ctx, "retention.o")
