"""Grouped-query attention over the paged cache, as a mixer part.

Formulas (YuvGev00/mini-engine): ``q, k, v = x Wq^T, x Wk^T, x Wv^T`` without biases, q and k
normalised per head with one weight ``[head_dim]`` shared by all heads, then rotated, in
that order (src/mini_engine/model.py:97-118); new keys and values are written to the cache
first, then every query reads all its keys from the cache (src/mini_engine/attention.py:117-121);
query head ``h`` reads KV head ``h // (heads / kv_heads)``, scores are scaled by
``head_dim**-0.5``, the query at position ``p`` sees positions ``<= p``
(src/mini_engine/attention.py:84-86,160-175).

The three projections run as one product on the row-concatenated weight, which leaves every
output element's sum unchanged.  Per-head norm, rotation and the cache write are one kernel.
All sizes and constants are constructor arguments; the part does not know its model.

Options beyond that model, each switched on by the spec: no position encoding at all
(``position_encoding=None``); value heads of their own width (``value_dim``); a window that keeps
the first ``keep_first`` tokens of the sequence readable for good (query ``p`` sees key ``j <= p``
when ``p - j < window`` or ``j < keep_first``); a distance bias taken off the scores,
``r1[h] * ln(1 + r2[h] * (p - j))`` with two learned numbers per head (``distance_bias``); and the
heads' softmax weights mixed by a learned ``[heads, heads]`` matrix before they meet the values
(``talking_heads``: ``w'_h = sum_g T[h, g] w_g``, head ``h`` reads its own KV head with ``w'_h``).  The
last four run in the kernels of ``csrc/attention_biased.cu``.

Three more, for designs that normalise and gate differently: ``qk_norm_scope="projection"`` takes the
root mean square of q over *all* its heads at once, and of k over all of its, with weights of that size
(``"head"``, the default, is per head with one shared weight); ``softmax_sink`` adds a silent
participant of score zero and no value to every softmax, ``p_j = exp(s_j) / (1 + sum_i exp(s_i))``;
``head_gate`` multiplies head ``h``'s output by ``sigmoid(W_g x)_h`` with a learned ``W_g [heads,
hidden]`` that runs as extra rows of the fused q/k/v product.  A layer that reads another entry's cache
(``reads_shared_cache``) may have a window of its own.

And four for designs without rotation whose positions enter through the scores: ``distance_bias="linear"`` takes
``slope_h * (p - j)`` off the scaled score of query ``p`` and key ``j``, with the fixed slopes ``slope_h = 2 **
(-linear_bias_span * (h + 1) / heads)``; ``softmax_sink="learned"`` makes the silent participant's score a learned
number per head (tensor ``sink``), ``p_j = exp(s_j) / (exp(sink_h) + sum_i exp(s_i))``; ``element_gate`` multiplies
the concatenated heads element by element with ``sigmoid(W_g x)``, ``W_g [heads * value_dim, hidden]``, again as rows
of the fused product; ``o_bias`` gives the output projection a bias, which the block hands to the norm that adds
the projection's partial sums.  With these, ``qkv_bias`` may be combined.

And two for designs that normalise behind the rotation and bound their scores: ``unit_norm_eps`` divides every q and
k head, *after* its rotation, by its root mean square over ``head_dim`` (eps inside the root, no weight), in the
kernel that adds the biases, rotates and writes the cache; ``score_softcap`` replaces a scaled score ``s`` by ``cap *
tanh(s / cap)``.  They combine with ``qkv_bias``, ``value_dim``, ``scale``, a partial rotation and either sink.
"""

from __future__ import annotations

from typing import Any, Mapping

import torch

from mini_engine_b200.config.model_spec import PartSpec
from mini_engine_b200.csrc import ops
from mini_engine_b200.parts.base import (
    LayerCache,
    Mixer,
    PagedCacheSpec,
    StepContext,
    build_part,
    register,
)
from mini_engine_b200.parts.linear import Linear
from mini_engine_b200.weights.loader import WeightSpec


@register("mixer", "gqa_attention")
class GroupedQueryAttention(Mixer):
    capturable = True

    def __init__(
        self,
        prefix: str,
        hidden_size: int,
        *,
        num_heads: int,
        kv_heads: int,
        head_dim: int,
        position_encoding: PartSpec | None,
        qk_norm_eps: float | None = None,
        window: int | None = None,
        scale: float | None = None,
        reads_shared_cache: bool = False,
        qkv_bias: bool = False,
        names: Mapping[str, str] | None = None,
        value_dim: int | None = None,
        keep_first: int = 0,
        distance_bias: bool | str = False,
        talking_heads: bool = False,
        qk_norm_scope: str = "head",
        softmax_sink: bool | str = False,
        head_gate: bool = False,
        element_gate: bool = False,
        o_bias: bool = False,
        linear_bias_span: float = 8.0,
        unit_norm_eps: float | None = None,
        score_softcap: float | None = None,
    ):
        if num_heads % kv_heads:
            raise ValueError(f"num_heads ({num_heads}) must be a multiple of kv_heads ({kv_heads})")
        self.value_dim = head_dim if value_dim is None else int(value_dim)
        self.keep_first = int(keep_first) if window else 0
        if distance_bias not in (False, True, "log", "linear") or softmax_sink not in (False, True, "learned"):
            raise ValueError("distance_bias is False, 'log' or 'linear'; softmax_sink is False, True or 'learned'")
        self.linear_bias = distance_bias == "linear"
        self.linear_bias_span = float(linear_bias_span)
        self.learned_sink = softmax_sink == "learned"
        distance_bias = bool(distance_bias) and not self.linear_bias  # below: the logarithmic form with learned constants
        self.distance_bias, self.talking_heads = bool(distance_bias), bool(talking_heads)
        # Whether the step runs in the kernels that know these options (any head size) or in the plain ones.
        if qk_norm_scope not in ("head", "projection"):
            raise ValueError(f"qk_norm_scope must be 'head' or 'projection', got {qk_norm_scope!r}")
        self.wide_norm = qk_norm_scope == "projection" and qk_norm_eps is not None
        self.sink, self.head_gate, self.element_gate = bool(softmax_sink), bool(head_gate), bool(element_gate)
        if self.head_gate and self.element_gate:
            raise ValueError("a mixer gates its heads or its elements, not both")
        self.has_output_bias = bool(o_bias)
        self.unit_norm_eps = None if unit_norm_eps is None else float(unit_norm_eps)
        self.softcap = float(score_softcap) if score_softcap else 0.0
        if self.softcap < 0.0:
            raise ValueError(f"score_softcap must be positive, got {score_softcap}")
        # The kernel that adds biases, rotates, then divides by the root mean square: it stands where the other
        # stores would, in front of the attention kernels that know a sink and a cap.
        self.unit_store = self.unit_norm_eps is not None or bool(self.softcap)
        if self.unit_store and (qk_norm_eps is not None or head_gate or element_gate or distance_bias or talking_heads or keep_first or reads_shared_cache or o_bias):
            raise ValueError("unit_norm_eps and score_softcap do not combine with q/k norm weights, gates, distance biases, talking heads, keep_first, an output bias or a shared cache")
        # Whether q, k, v (and the gates) leave the fused product through the kernel that normalises whole projections.
        self.wide_store = self.wide_norm or self.head_gate or self.element_gate or self.linear_bias
        if (self.head_gate or self.element_gate or self.linear_bias) and qk_norm_eps is not None and not self.wide_norm:
            raise ValueError("gates and the linear distance bias come with qk_norm_scope='projection' or without q/k norms")
        if (self.wide_store or self.sink) and (keep_first or distance_bias or talking_heads):
            raise ValueError("qk_norm_scope='projection', softmax_sink, gates and the linear distance bias do not combine with keep_first, the logarithmic distance_bias or talking_heads")
        if qkv_bias and self.sink and not self.wide_store and not self.unit_store:
            raise ValueError("biases with a sink need the projection-wide store (a gate, a linear bias or qk_norm_scope='projection')")
        self.extended = bool(
            (self.value_dim != head_dim and not (self.wide_store or self.sink or self.unit_store)) or self.keep_first or distance_bias or talking_heads
        )
        if self.extended:
            if reads_shared_cache or qkv_bias:
                raise ValueError("the extended attention options do not combine with a shared cache or biases")
            if head_dim < 1 or self.value_dim < 1 or keep_first < 0:
                raise ValueError("head sizes must be positive and keep_first must not be negative")
        elif self.wide_store or self.sink or self.unit_store:  # these run in the kernel that takes any head size
            if not (1 <= head_dim <= 512 and 1 <= self.value_dim <= 512):
                raise ValueError(f"head sizes must lie between 1 and 512, got {head_dim} and {self.value_dim}")
        else:
            ops.check_attention_sizes(head_dim, num_heads, kv_heads)
        self.hidden, self.heads, self.kv_heads, self.head_dim = hidden_size, num_heads, kv_heads, head_dim
        self.qk_norm_eps = qk_norm_eps
        self.window = window
        # Mixed heads under a window run as two kernels that keep the scores of the (bounded) visible keys, when
        # the sizes fit them (and, decided per engine in `forward`, the scratch stays under 2 GiB); else in one pass.
        self.two_kernel_mixing = bool(
            self.talking_heads and window
            and num_heads // kv_heads <= ops.MIXED_ATTENTION_MAX_GROUP and self.value_dim <= ops.MIXED_ATTENTION_MAX_VALUE_DIM
        )  # fmt: skip
        self.scale = float(scale) if scale is not None else head_dim**-0.5
        self.reads_shared_cache = reads_shared_cache
        self.qkv_bias = qkv_bias  # the reference's projections have none (src/mini_engine/model.py:97-100)
        defaults = {
            "q": "q_proj.weight",
            "k": "k_proj.weight",
            "v": "v_proj.weight",
            "o": "o_proj.weight",
            "q_norm": "q_norm.weight",
            "k_norm": "k_norm.weight",
            "q_bias": "q_proj.bias",
            "k_bias": "k_proj.bias",
            "v_bias": "v_proj.bias",
            "r1": "distance_bias.r1",
            "r2": "distance_bias.r2",
            "talk": "talking_heads.weight",
            "gate": "gate_proj.weight",
            "sink": "sink",
            "o_bias": "o_proj.bias",
        }
        self.names = {key: prefix + (names or {}).get(key, value) for key, value in defaults.items()}
        self.position = None
        if position_encoding is not None:
            self.position = build_part("position_encoding", position_encoding, prefix, hidden_size)
        self.r1 = self.r2 = self.talk = None
        self.gates = num_heads if self.head_gate else num_heads * self.value_dim if self.element_gate else 0
        self.slopes: torch.Tensor | None = None
        self.sink_values: torch.Tensor | None = None
        self.qkv: Linear | None = None
        self.out: Linear | None = None
        self.q_norm: torch.Tensor | None = None
        self.k_norm: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None

    # ------------------------------------------------------------------ declarations

    def paged_cache(self) -> PagedCacheSpec:
        value_dim = None if self.value_dim == self.head_dim else self.value_dim
        return PagedCacheSpec(self.kv_heads, self.head_dim, self.window, value_dim, self.keep_first)

    def weight_specs(self) -> list[WeightSpec]:
        d, n = self.head_dim, self.names
        specs = [WeightSpec(n["q"], (self.heads * d, self.hidden))]
        if not self.reads_shared_cache:
            specs += [
                WeightSpec(n["k"], (self.kv_heads * d, self.hidden)),
                WeightSpec(n["v"], (self.kv_heads * self.value_dim, self.hidden)),
            ]
        specs.append(WeightSpec(n["o"], (self.hidden, self.heads * self.value_dim)))
        if self.distance_bias:
            specs += [WeightSpec(n[key], (self.heads,), role="vector", init="positive") for key in ("r1", "r2")]
        if self.talking_heads:
            specs.append(WeightSpec(n["talk"], (self.heads, self.heads), role="vector", init="ones_normal"))
        if self.gates:
            specs.append(WeightSpec(n["gate"], (self.gates, self.hidden)))
        if self.learned_sink:
            specs.append(WeightSpec(n["sink"], (self.heads,), role="vector", init="wide_normal"))
        if self.has_output_bias:
            specs.append(WeightSpec(n["o_bias"], (self.hidden,), role="vector", init="small_normal"))
        if self.qk_norm_eps is not None:
            q_len, k_len = (self.heads * d, self.kv_heads * d) if self.wide_norm else (d, d)
            specs.append(WeightSpec(n["q_norm"], (q_len,), role="vector", init="ones_normal"))
            if not self.reads_shared_cache:
                specs.append(WeightSpec(n["k_norm"], (k_len,), role="vector", init="ones_normal"))
        if self.qkv_bias:
            specs.append(WeightSpec(n["q_bias"], (self.heads * d,), role="vector"))
            if not self.reads_shared_cache:
                specs.append(WeightSpec(n["k_bias"], (self.kv_heads * d,), role="vector"))
                specs.append(WeightSpec(n["v_bias"], (self.kv_heads * self.value_dim,), role="vector"))
        return specs + (self.position.weight_specs() if self.position is not None else [])

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        rows = [tensors[n["q"]]]
        if not self.reads_shared_cache:
            rows += [tensors[n["k"]], tensors[n["v"]]]
        if self.gates:
            rows.append(tensors[n["gate"]])
        self.qkv = Linear(torch.cat(rows, dim=0).contiguous() if len(rows) > 1 else rows[0])
        self.out = Linear(tensors[n["o"]])
        if self.qk_norm_eps is not None:
            self.q_norm = tensors[n["q_norm"]]
            self.k_norm = None if self.reads_shared_cache else tensors[n["k_norm"]]
        if self.qkv_bias:
            parts = [tensors[n["q_bias"]]]
            if not self.reads_shared_cache:
                parts += [tensors[n["k_bias"]], tensors[n["v_bias"]]]
            if self.gates:  # the gate rows of the fused product have no bias
                parts.append(torch.zeros(self.gates, dtype=parts[0].dtype, device=parts[0].device))
            self.bias = torch.cat(parts).contiguous()
        if self.has_output_bias:
            self.output_bias = tensors[n["o_bias"]]
        if self.learned_sink:
            self.sink_values = tensors[n["sink"]]
        if self.linear_bias:
            slopes = [2.0 ** (-self.linear_bias_span * (h + 1) / self.heads) for h in range(self.heads)]
            self.slopes = torch.tensor(slopes, dtype=torch.float32, device=tensors[n["q"]].device)
        if self.distance_bias:
            self.r1, self.r2 = tensors[n["r1"]], tensors[n["r2"]]
        if self.talking_heads:
            self.talk = tensors[n["talk"]]
        if self.position is not None:
            self.position.load(tensors)

    # ------------------------------------------------------------------------ step

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        tokens, d = h.shape[0], self.head_dim
        kv_in = 0 if self.reads_shared_cache else self.kv_heads
        qkv = self.qkv.forward(h, ctx, "attn.qkv")
        q = ctx.buffer("attn.q", (tokens, self.heads * d), ctx.dtype)
        table = self.position.step_angles(ctx) if self.position is not None else None
        slots = ctx.slot_mapping[cache.group]
        if self.unit_store:
            return self._forward_unit(qkv, q, table, slots, ctx, cache)
        if self.wide_store or self.sink:
            return self._forward_gated(qkv, q, table, slots, ctx, cache)
        args: dict[str, Any] = dict(
            qkv=qkv, heads=self.heads, kv_heads=kv_in, head_dim=d, q_weight=self.q_norm,
            k_weight=self.k_norm, eps=self.qk_norm_eps or 0.0, positions=ctx.positions, q_out=q,
            page_size=ctx.page_size, bias=self.bias, value_dim=self.value_dim,
        )  # fmt: skip
        if kv_in and not cache.writes:
            # This execution reads another entry's cache: its own keys and values are not kept.
            unused_k = ctx.buffer("attn.k_new", (tokens, kv_in * d), ctx.dtype)
            unused_v = ctx.buffer("attn.v_new", (tokens, kv_in * d), ctx.dtype)
            ops.qk_norm_rope_store(**args, cos_sin=table, k_dense=unused_k, v_dense=unused_v)
            if table is None and self.position is not None:
                self.position.apply(q.view(tokens, self.heads, d), unused_k.view(tokens, kv_in, d), ctx.positions)
        elif table is not None or kv_in == 0 or self.position is None:
            ops.qk_norm_rope_store(
                **args, cos_sin=table, slot_mapping=slots, k_pages=cache.k, v_pages=cache.v
            )
        else:  # a position encoding that the fused kernel does not know: three steps
            k_new = ctx.buffer("attn.k_new", (tokens, kv_in * d), ctx.dtype)
            v_new = ctx.buffer("attn.v_new", (tokens, kv_in * d), ctx.dtype)
            ops.qk_norm_rope_store(**args, cos_sin=None, k_dense=k_new, v_dense=v_new)
            self.position.apply(q.view(tokens, self.heads, d), k_new.view(tokens, kv_in, d), ctx.positions)
            ops.kv_store(k_new, v_new, slots, cache.k, cache.v, kv_in, d, ctx.page_size)
        if self.extended:
            out = ctx.buffer("attn.out", (tokens, self.heads * self.value_dim), ctx.dtype)
            # Scores of every visible key are kept between two kernels; a window bounds them whatever the context.
            # The scratch is sized for the engine's token capacity, so the choice never depends on the batch.
            stride = (self.window or 0) + self.keep_first
            capacity = max(tokens, ctx.workspace.max_tokens)
            if self.two_kernel_mixing and capacity * self.heads * stride * 4 <= 2 << 30:
                scores = ctx.buffer("attn.scores", (tokens, self.heads * stride), torch.float32)
                stats = ctx.buffer("attn.stats", (tokens, self.heads * 2), torch.float32)
                ops.mixed_attention(
                    q=q, k_pages=cache.k, v_pages=cache.v, block_table=ctx.block_tables[cache.group],
                    entry_of_token=ctx.entry_of_token, positions=ctx.positions, out=out, heads=self.heads,
                    kv_heads=self.kv_heads, head_dim=d, value_dim=self.value_dim, scale=self.scale, window=self.window,
                    keep_first=self.keep_first, r1=self.r1, r2=self.r2, talk=self.talk, scores=scores, stats=stats,
                    stride=stride,
                )  # fmt: skip
                return self.out.forward(out, ctx, "attn.o")
            spread = None
            if self.talk is not None:
                spread = ctx.buffer("attn.spread", (tokens, self.heads * self.kv_heads * self.value_dim), torch.float32)
            ops.biased_attention(
                q=q, k_pages=cache.k, v_pages=cache.v, block_table=ctx.block_tables[cache.group],
                entry_of_token=ctx.entry_of_token, positions=ctx.positions, out=out, heads=self.heads,
                kv_heads=self.kv_heads, head_dim=d, value_dim=self.value_dim, scale=self.scale,
                window=self.window or 0, keep_first=self.keep_first, r1=self.r1, r2=self.r2, talk=self.talk,
                spread=spread,
            )  # fmt: skip
            return self.out.forward(out, ctx, "attn.o")
        out = ctx.buffer("attn.out", (tokens, self.heads * d), ctx.dtype)
        ops.paged_attention(
            q=q, k_pages=cache.k, v_pages=cache.v, block_table=ctx.block_tables[cache.group], ctx=ctx,
            out=out, heads=self.heads, kv_heads=self.kv_heads, head_dim=d, scale=self.scale,
            window=self.window or 0,
        )  # fmt: skip
        return self.out.forward(out, ctx, "attn.o")

    def _forward_unit(self, qkv, q, table, slots, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        """The step with q and k normalised behind their rotation and (or) capped scores."""
        tokens = q.shape[0]
        if self.position is not None and table is None:
            raise ValueError("these attention options take a rotation that the fused kernel applies, or none")
        ops.qkv_rope_unit_store(
            qkv=qkv, heads=self.heads, kv_heads=self.kv_heads, head_dim=self.head_dim, value_dim=self.value_dim,
            bias=self.bias, cos_sin=table, unit_norm_eps=self.unit_norm_eps, q_out=q, page_size=ctx.page_size,
            slot_mapping=slots, k_pages=cache.k, v_pages=cache.v,
        )  # fmt: skip
        out = ctx.buffer("attn.out", (tokens, self.heads * self.value_dim), ctx.dtype)
        ops.paged_attention(
            q=q, k_pages=cache.k, v_pages=cache.v, block_table=ctx.block_tables[cache.group], ctx=ctx, out=out,
            heads=self.heads, kv_heads=self.kv_heads, head_dim=self.head_dim, scale=self.scale, window=self.window or 0,
            value_dim=self.value_dim, sink=self.sink, sink_values=self.sink_values, softcap=self.softcap,
        )  # fmt: skip
        return self.out.forward(out, ctx, "attn.o")

    def _forward_gated(self, qkv, q, table, slots, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        """The step with a projection-wide norm, a sink in the softmax or gated heads."""
        tokens, d = q.shape[0], self.head_dim
        kv_in = 0 if self.reads_shared_cache else self.kv_heads
        if self.position is not None and table is None:
            raise ValueError("these attention options take a rotation that the fused kernel applies, or none")
        gate = ctx.buffer("attn.gate", (tokens, self.gates), torch.float32) if self.gates else None
        if self.wide_store:
            args: dict[str, Any] = dict(
                qkv=qkv, heads=self.heads, kv_heads=kv_in, head_dim=d, value_dim=self.value_dim, q_weight=self.q_norm,
                k_weight=self.k_norm, eps=self.qk_norm_eps or 0.0, cos_sin=table, q_out=q, page_size=ctx.page_size,
                gates=self.gates, gate_out=gate, bias=self.bias,
            )  # fmt: skip
            if kv_in and not cache.writes:  # this execution reads another entry's cache: its own keys and values are not kept
                unused_k = ctx.buffer("attn.k_new", (tokens, kv_in * d), ctx.dtype)
                unused_v = ctx.buffer("attn.v_new", (tokens, kv_in * self.value_dim), ctx.dtype)
                ops.qk_wide_norm_rope_store(**args, k_dense=unused_k, v_dense=unused_v)
            else:
                ops.qk_wide_norm_rope_store(**args, slot_mapping=slots, k_pages=cache.k, v_pages=cache.v)
        else:
            ops.qk_norm_rope_store(
                qkv=qkv, heads=self.heads, kv_heads=kv_in, head_dim=d, q_weight=self.q_norm, k_weight=self.k_norm,
                eps=self.qk_norm_eps or 0.0, positions=ctx.positions, q_out=q, page_size=ctx.page_size, cos_sin=table,
                value_dim=self.value_dim, slot_mapping=slots, k_pages=cache.k, v_pages=cache.v,
            )  # fmt: skip
        out = ctx.buffer("attn.out", (tokens, self.heads * self.value_dim), ctx.dtype)
        ops.paged_attention(
            q=q, k_pages=cache.k, v_pages=cache.v, block_table=ctx.block_tables[cache.group], ctx=ctx, out=out,
            heads=self.heads, kv_heads=self.kv_heads, head_dim=d, scale=self.scale, window=self.window or 0,
            value_dim=self.value_dim, sink=self.sink, gate=gate, slopes=self.slopes, sink_values=self.sink_values,
        )  # fmt: skip
        return self.out.forward(out, ctx, "attn.o")
