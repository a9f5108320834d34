"""Attention through a low-rank latent, as a mixer part.

Queries go through a latent of their own: ``c_q = rmsnorm(W_dq x)``, ``q = W_uq c_q``, laid out head by head as
``[dim plain | rot_dim rotated]``.  Keys and values come from one latent per token: ``W_dkv x`` has ``kv_rank +
rot_dim`` rows; the first ``kv_rank``, RMS-normed, are the latent ``c``; the last ``rot_dim`` are one rotated key
part ``k_r`` that all heads share.  Head ``h`` has the plain key ``U_k,h c`` and the value ``U_v,h c``, and

    score_h(i, j) = (q_plain_h(i) . U_k,h c_j + rot(q_rot_h(i)) . rot(k_r(j))) * scale.

Only ``[c | rot(k_r)]`` is cached, one row of ``kv_rank + rot_dim`` per token, and the two maps are applied on the
query's side: ``q'_h = [U_k,h^T q_plain_h | rot(q_rot_h)]`` meets the cached rows directly, the softmax weights
average ``c`` itself, and ``U_v,h`` is applied to that average.  So the attention kernel sees one shared key/value
head whose values are the first ``kv_rank`` elements of its keys (``PagedCacheSpec.value_dim == 0``).  Options: a
sliding ``window``, a ``scale``, and ``head_gate`` (head ``h``'s output times ``sigmoid(W_g x)_h``, ``W_g [heads,
hidden]``; it runs as rows of the fused down projection and is applied before ``U_v``, with which it commutes).

A step is: one product for ``[W_dq; W_dkv; W_g]``; a kernel that normalises both latents, rotates ``k_r``, writes the
cache row and forms the gates; the product ``W_uq``; a per-head product that forms ``q'`` (and rotates its last
part); attention; a per-head product with ``U_v``; the output projection.  Statistics, angles, scores, softmax and
gates are 32-bit.
"""

from __future__ import annotations

from typing import Mapping

import torch

from mini_engine_b200.config.model_spec import PartSpec
from mini_engine_b200.csrc import ops
from mini_engine_b200.parts.base import LayerCache, Mixer, PagedCacheSpec, StepContext, build_part, register
from mini_engine_b200.parts.linear import Linear
from mini_engine_b200.weights.loader import WeightSpec


@register("mixer", "latent_attention")
class LatentAttention(Mixer):
    capturable = True

    def __init__(
        self,
        prefix: str,
        hidden_size: int,
        *,
        num_heads: int,
        head_dim: int,
        rot_dim: int,
        value_dim: int,
        kv_rank: int,
        q_rank: int | None,
        norm_eps: float,
        scale: float | None = None,
        window: int | None = None,
        position_encoding: PartSpec | None = None,
        head_gate: bool = False,
        names: Mapping[str, str] | None = None,
        rotary_layout: str = "half",
    ):
        """``head_dim``: plain query/key elements per head; ``rot_dim``: rotated ones (0: none); ``position_encoding``
        must be a rotate-half rotation over at most ``rot_dim`` elements (or ``None``: the part is used as it is).
        ``q_rank=None``: the queries have no latent of their own, ``q = W_q x`` (tensor ``q``).  ``rotary_layout``
        ``"interleaved"``: the checkpoint pairs element ``2 i`` of a rotated part with ``2 i + 1``; the rows of the
        query and key projections that make the rotated parts are then reordered once, when they are loaded, to
        ``[even elements | odd elements]``: the same permutation on both sides leaves every score as it was, and the
        kernels rotate halves."""
        if rotary_layout not in ("half", "interleaved"):
            raise ValueError(f"rotary_layout is 'half' or 'interleaved', got {rotary_layout!r}")
        self.interleaved = rotary_layout == "interleaved"
        q_rank = int(q_rank or 0)
        if min(num_heads, head_dim, value_dim, kv_rank) < 1 or rot_dim < 0 or q_rank < 0:
            raise ValueError("latent_attention: sizes must be positive (rot_dim may be 0)")
        if value_dim > 512 or kv_rank > 512 or kv_rank + rot_dim > 2048:
            raise ValueError("latent_attention: kv_rank and value_dim up to 512, kv_rank + rot_dim up to 2048")
        self.hidden, self.heads, self.dim, self.rot_dim = hidden_size, num_heads, head_dim, rot_dim
        self.value_dim, self.kv_rank, self.q_rank = value_dim, kv_rank, q_rank
        self.eps = float(norm_eps)
        self.scale = float(scale) if scale is not None else (head_dim + rot_dim) ** -0.5
        self.window = window
        self.head_gate = bool(head_gate)
        self.position = None
        if position_encoding is not None:
            if rot_dim < 2:
                raise ValueError("latent_attention: a position encoding needs a rotated part")
            self.position = build_part("position_encoding", position_encoding, prefix, hidden_size)
        defaults = {
            "dq": "q_down.weight", "q_norm": "q_norm.weight", "uq": "q_up.weight", "dkv": "kv_down.weight",
            "kv_norm": "kv_norm.weight", "uk": "k_up.weight", "uv": "v_up.weight", "gate": "gate_proj.weight",
            "o": "o_proj.weight", "q": "q_proj.weight",
        }  # fmt: skip
        self.names = {key: prefix + (names or {}).get(key, value) for key, value in defaults.items()}
        self.down: Linear | None = None
        self.up_q: Linear | None = None
        self.out: Linear | None = None
        self.q_norm = self.kv_norm = self.key_maps = self.value_maps = None

    # ------------------------------------------------------------------ declarations

    def paged_cache(self) -> PagedCacheSpec:
        return PagedCacheSpec(1, self.kv_rank + self.rot_dim, self.window, value_dim=0)

    def weight_specs(self) -> list[WeightSpec]:
        n, heads = self.names, self.heads
        specs = [
            WeightSpec(n["dq"], (self.q_rank, self.hidden)),
            WeightSpec(n["q_norm"], (self.q_rank,), role="vector", init="ones_normal"),
            WeightSpec(n["uq"], (heads * (self.dim + self.rot_dim), self.q_rank)),
        ] if self.q_rank else [WeightSpec(n["q"], (heads * (self.dim + self.rot_dim), self.hidden))]
        specs += [
            WeightSpec(n["dkv"], (self.kv_rank + self.rot_dim, self.hidden)),
            WeightSpec(n["kv_norm"], (self.kv_rank,), role="vector", init="ones_normal"),
            WeightSpec(n["uk"], (heads * self.dim, self.kv_rank)),
            WeightSpec(n["uv"], (heads * self.value_dim, self.kv_rank)),
        ]
        if self.head_gate:
            specs.append(WeightSpec(n["gate"], (heads, self.hidden)))
        specs.append(WeightSpec(n["o"], (self.hidden, heads * self.value_dim)))
        return specs + (self.position.weight_specs() if self.position is not None else [])

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        down_kv, up_q = tensors[n["dkv"]], tensors[n["uq"] if self.q_rank else n["q"]]
        if self.interleaved and self.position is not None:
            dims = self.position.rotary_dim
            order = torch.cat((torch.arange(0, dims, 2), torch.arange(1, dims, 2), torch.arange(dims, self.rot_dim))).to(up_q.device)
            per_head = up_q.view(self.heads, self.dim + self.rot_dim, -1)
            up_q = torch.cat((per_head[:, : self.dim], per_head[:, self.dim :][:, order]), dim=1).reshape(up_q.shape).contiguous()
            down_kv = torch.cat((down_kv[: self.kv_rank], down_kv[self.kv_rank :][order]), dim=0).contiguous()
        rows = ([tensors[n["dq"]]] if self.q_rank else []) + [down_kv]
        if self.head_gate:
            rows.append(tensors[n["gate"]])
        self.down = Linear(torch.cat(rows, dim=0).contiguous() if len(rows) > 1 else rows[0])
        self.up_q = Linear(up_q)  # without a query latent: the query projection itself
        self.out = Linear(tensors[n["o"]])
        self.q_norm, self.kv_norm = (tensors[n["q_norm"]] if self.q_rank else None), tensors[n["kv_norm"]]
        # U_k as stored is [heads][dim][kv_rank]: the map from a head's plain query to the latent's space.
        self.key_maps = tensors[n["uk"]].view(self.heads, self.dim, self.kv_rank)
        # U_v as stored is [heads][value_dim][kv_rank]; the kernel walks the inner index first.
        self.value_maps = tensors[n["uv"]].view(self.heads, self.value_dim, self.kv_rank).transpose(1, 2).contiguous()
        if self.position is not None:
            self.position.load(tensors)

    # ------------------------------------------------------------------------ step

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        tokens, heads = h.shape[0], self.heads
        key_width = self.kv_rank + self.rot_dim
        table = self.position.step_angles(ctx) if self.position is not None else None
        if self.position is not None and table is None:
            raise ValueError("latent_attention takes a rotation that its kernels apply, or none")
        down = self.down.forward(h, ctx, "latent.down")
        q_latent = ctx.buffer("latent.q_latent", (tokens, self.q_rank), ctx.dtype) if self.q_rank else None
        gate = ctx.buffer("latent.gate", (tokens, heads), torch.float32) if self.head_gate else None
        ops.latent_down_finish(
            down=down, q_rank=self.q_rank, kv_rank=self.kv_rank, rot_dim=self.rot_dim, q_weight=self.q_norm,
            kv_weight=self.kv_norm, eps=self.eps, cos_sin=table, slot_mapping=ctx.slot_mapping[cache.group],
            q_latent=q_latent, k_pages=cache.k, gates=heads if self.head_gate else 0, gate_out=gate,
        )  # fmt: skip
        q_parts = self.up_q.forward(q_latent if self.q_rank else h, ctx, "latent.q")
        q = ctx.buffer("latent.q_mapped", (tokens, heads * key_width), ctx.dtype)
        ops.head_product(q_parts, self.key_maps, q, tail=self.rot_dim, cos_sin=table)
        mean = ctx.buffer("latent.mean", (tokens, heads * self.kv_rank), ctx.dtype)
        ops.paged_attention(
            q=q, k_pages=cache.k, v_pages=None, block_table=ctx.block_tables[cache.group], ctx=ctx, out=mean,
            heads=heads, kv_heads=1, head_dim=key_width, scale=self.scale, window=self.window or 0,
            value_dim=self.kv_rank, gate=gate,
        )  # fmt: skip
        out = ctx.buffer("latent.out", (tokens, heads * self.value_dim), ctx.dtype)
        ops.head_product(mean, self.value_maps, out)
        return self.out.forward(out, ctx, "latent.o")
