"""Interfaces and registries of the parts a layer is made of.

A layer is assembled from parts and an arrangement:

* a **mixer** (token mixing: attention here) that may keep per-token pages and/or a
  fixed-size per-request state in the cache manager,
* a **feed-forward**,
* **norms**, by the names that the arrangement asks for (two in a pre-norm layer),
* a **block** that says how they are wired (pre-norm residual here),

and a mixer may own a **position encoding**.  The model's two ends are parts as well: an
**embedding** and a **head**.  Each kind has one registry from a name to a
class; a :class:`~mini_engine_b200.config.model_spec.PartSpec` names the class and carries
its constants.  No part reads a model configuration or knows which model it is in.

The hidden state travels as a :class:`Residual`: the 32-bit residual stream plus the
not-yet-added output of the previous part.  A norm adds the pending output while it
normalises, which fuses the residual sum (in 32-bit) with the next norm's read.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Mapping

import torch

from mini_engine_b200.config.model_spec import PartSpec
from mini_engine_b200.weights.loader import WeightSpec

# ------------------------------------------------------------------------------ cache needs


@dataclass(frozen=True)
class PagedCacheSpec:
    """Per-token cache of one mixer: K and V of ``kv_heads`` heads of ``head_dim`` values.

    ``window`` is ``None`` when every key is kept; else only the last ``window`` positions
    are ever read and pages wholly behind the window are given back while the request runs.
    With a window, ``keep_first`` tokens at the start of the sequence stay readable for good (their
    pages are never given back).  ``value_dim`` is the width of a value head when it differs from
    ``head_dim``; 0 says that the values are a part of the key rows (a cache of one latent row per token
    that serves as key and as value), so that no value pages are kept.  Mixers with an equal spec share
    one cache group (one page pool, one block table per request).
    """

    kv_heads: int
    head_dim: int
    window: int | None = None
    value_dim: int | None = None
    keep_first: int = 0

    @property
    def v_dim(self) -> int:
        return self.head_dim if self.value_dim is None else self.value_dim


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size: ``shape`` elements of ``dtype`` per request."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


# ------------------------------------------------------------------------- step-time data


@dataclass
class Residual:
    """The residual stream ``x [T, hidden]`` (float32) and a pending addend.

    ``pending`` is ``None`` or a float32 tensor ``[S, T, hidden]`` whose ``S`` slices (the
    partial sums of a split matrix product) are all still to be added to ``x``; with
    ``pending_scale`` (float32 ``[hidden]``, a layer scale) their sum is multiplied column by column
    before it is added.  ``rounded`` is ``x`` in the compute dtype when a part has already made that
    copy (an embedding, or a norm that wrote its result back to ``x``), for a sublayer that reads the
    stream itself; whoever changes ``x`` sets or clears it.  ``pending_bias`` (float32 ``[hidden]``) is the
    bias of the output projection whose partial sums are pending, added with them.  ``pending_more`` is
    the output of a second sublayer that read the same input as the first (sublayers side by side),
    ``[S', T, hidden]``, added as well.  A norm that does not know one of these must refuse it.

    A model with several residual streams (hyper-connections) keeps them in ``streams [N, T, hidden]`` (float32)
    beside ``x``, which then holds the embedding's output: until the first update has been written
    (``streams_unwritten``) every stream equals ``x``.  ``stream_update`` says how the pending output enters the
    streams, ``(mix [N, N], share [N], mult)``: ``x_t = sum_s mix[s, t] x_s + mult * share[t] * pending``;
    ``stream_read [N]`` are the weights of the sum that the next norm normalises (``None``: all ones, the model's
    end).  The norm applies the update, writes the streams back and reads them in one kernel.
    """

    x: torch.Tensor
    pending: torch.Tensor | None = None
    pending_scale: torch.Tensor | None = None
    rounded: torch.Tensor | None = None
    pending_bias: torch.Tensor | None = None
    pending_more: torch.Tensor | None = None
    streams: torch.Tensor | None = None
    streams_unwritten: bool = False
    stream_update: tuple | None = None
    stream_read: torch.Tensor | None = None

    def add(self, delta: torch.Tensor, scale: torch.Tensor | None = None, bias: torch.Tensor | None = None) -> None:
        if self.pending is not None:
            raise RuntimeError("a pending output must be consumed by a norm before the next is set")
        if delta.dim() == 2:
            delta = delta.unsqueeze(0)
        self.pending, self.pending_scale, self.pending_bias = delta, scale, bias

    def add_beside(self, delta: torch.Tensor) -> None:
        """The output of a sublayer that ran beside the one whose output is pending."""
        if self.pending is None or self.pending_more is not None or self.pending_scale is not None:
            raise RuntimeError("a second output goes beside exactly one pending output without a scale")
        self.pending_more = delta.unsqueeze(0) if delta.dim() == 2 else delta

    def clear(self) -> None:
        self.pending = self.pending_scale = self.pending_bias = self.pending_more = None
        self.stream_update = self.stream_read = None


@dataclass
class LayerCache:
    """What one execution of a mixer sees of the cache.

    ``k`` and ``v`` are the page arrays of this entry, ``[pages + 1, kv_heads, page_size,
    head_dim]`` (the last page is a spare that no request owns); ``group`` indexes the
    per-group arrays of :class:`StepContext`; ``writes`` is False when the entry reads
    another entry's cache.  ``state`` is ``[slots + 1, *StateSpec.shape]`` or ``None``.
    """

    group: int | None = None
    k: torch.Tensor | None = None
    v: torch.Tensor | None = None
    writes: bool = True
    state: torch.Tensor | None = None


@dataclass
class StepContext:
    """One batch of (request, its next tokens), flattened; all index tensors are int32.

    Tokens of all entries are concatenated in entry order.  Entry ``b`` owns tokens
    ``cu_tokens[b] .. cu_tokens[b+1]``, which are the positions ``context_lens[b] - n_b ..
    context_lens[b] - 1`` of its request.
    """

    dtype: torch.dtype  # compute dtype of matrices and activations
    num_tokens: int
    num_entries: int
    max_query_len: int
    max_context_len: int
    token_ids: torch.Tensor  # [T]
    positions: torch.Tensor  # [T] absolute position of each token in its request
    entry_of_token: torch.Tensor  # [T]
    cu_tokens: torch.Tensor  # [B + 1]
    context_lens: torch.Tensor  # [B] tokens of the request after this step
    state_slots: torch.Tensor  # [B] slot of the request's fixed-size state
    fresh: torch.Tensor  # [B] 1 when the entry starts at position 0 (state starts from zero)
    slot_mapping: list[torch.Tensor] = field(default_factory=list)  # per group [T]: page * page_size + offset
    block_tables: list[torch.Tensor] = field(default_factory=list)  # per group [B, max_blocks]
    page_size: int = 16
    workspace: "Any" = None  # Workspace: named persistent buffers
    all_decode: bool = False  # every entry brings exactly one token
    num_decode_entries: int = 0  # entries that bring exactly one token ...
    decode_entries: torch.Tensor | None = None  # ... their numbers, ascending (int32)
    portion_entries: torch.Tensor | None = None  # the numbers of the entries that bring more
    host: Mapping[str, Any] = field(default_factory=dict)  # host copies for parts written in Python
    embedding_state: torch.Tensor | None = None  # [slots + 1, *shape]: per-request state of the embedding part
    memo: dict = field(default_factory=dict)  # what parts compute once per step and share between layers

    def buffer(self, name: str, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        return self.workspace.get(name, shape, dtype)


# ------------------------------------------------------------------------------ interfaces


class Part:
    """Common to all parts: declared weights and their arrival."""

    # Whether the part's launches depend on the batch through device arrays and the token count
    # alone, so that a step of a fixed token count can be captured in a CUDA graph and replayed for
    # other requests (a part whose Python reads ``ctx.host`` or branches on values must say False).
    capturable = False
    # Whether a step of a model with this part may launch its kernels as programmatic dependents of one
    # another (CTAs of a kernel resident while its predecessor still runs).  A part says False when steps
    # with its kernels were seen to stall that way; the whole step then runs in plain stream order.
    programmatic_launch = True

    def weight_specs(self) -> list[WeightSpec]:
        return []

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Receive the declared tensors (already on the device, cast by role)."""


class Norm(Part):
    def forward(
        self,
        state: Residual,
        ctx: StepContext,
        out_dtype: torch.dtype,
        rows: torch.Tensor | None = None,
        residual_scale: float = 1.0,
        keep_normed: bool = False,
    ) -> torch.Tensor:
        """Add ``state.pending`` into ``state.x`` (and clear it), return the normalised rows
        in ``out_dtype``.  With ``rows`` (int32 ``[N]``) only those rows are produced, as
        ``[N, hidden]``, and ``state.x`` is left as it was.  ``residual_scale`` multiplies ``state.x``
        before the pending output is added; with ``keep_normed`` the normalised rows (float32) replace
        ``state.x`` (an arrangement whose norm follows the sum)."""
        raise NotImplementedError


class PositionEncoding(Part):
    def fused_rotary_table(self) -> torch.Tensor | None:
        """Inverse frequencies ``[rotary_dim / 2]`` (float32, on the device) when the
        encoding is a rotate-half rotation that the mixer's fused kernel can apply; else
        ``None`` and the mixer calls :meth:`apply`."""
        return None

    def step_angles(self, ctx: "StepContext") -> torch.Tensor | None:
        """``[T, rotary_dim / 2, 2]`` float32 (cos, sin) for the step's tokens when the
        encoding is a fusable rotation, made once per step and shared by all layers."""
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        """Encode positions in place into ``q [T, heads, d]`` and ``k [T, kv_heads, d]``.
        Keys are cached after this call, so the encoding may depend on the absolute
        position only."""
        raise NotImplementedError


class Mixer(Part):
    # The bias of the mixer's output projection (float32 ``[hidden]``) when it has one: `forward` returns the
    # product's partial sums without it, and the block hands it to the norm that adds them (``Residual.add``).
    # A block that does not (``Block.adds_output_bias``) cannot hold such a mixer.
    output_bias: torch.Tensor | None = None
    has_output_bias = False

    def paged_cache(self) -> PagedCacheSpec | None:
        return None

    def state(self) -> StateSpec | None:
        return None

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        """``h [T, hidden]`` (compute dtype) -> output ``[S, T, hidden]`` float32 whose ``S``
        slices sum to the mixer's output."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        """``h [T, hidden]`` -> ``[S, T, hidden]`` float32, as for a mixer."""
        raise NotImplementedError


class Embedding(Part):
    """The model's first part: token ids to rows of the residual stream."""

    def state(self) -> StateSpec | None:
        """Per-request state of fixed size that the embedding keeps between steps (``ctx.embedding_state``,
        indexed by the request's state slot), or ``None``."""
        return None

    def forward(self, token_ids: torch.Tensor, ctx: StepContext, out: torch.Tensor) -> torch.Tensor | None:
        """Fill ``out [T, hidden]`` (float32, the residual stream) for ``token_ids [T]`` (int32).  May
        return the same rows in the compute dtype when it has made them on the way."""
        raise NotImplementedError


class Head(Part):
    """The model's last part: normalised rows to logits."""

    def forward(self, rows: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        """``rows [N, hidden]`` (compute dtype) -> float32 logits ``[N, vocab]``."""
        raise NotImplementedError


class Block(Part):
    """Arrangement of mixer, feed-forward and norms around the residual stream.

    ``NORMS`` lists the names of the norms that the arrangement uses; the layer's spec must give
    exactly those (``LayerSpec.named_norms``), and they arrive as ``self.norms[name]``."""

    NORMS: tuple[str, ...] = ("mixer", "feed_forward")
    adds_output_bias = False  # whether the arrangement hands `Mixer.output_bias` on with the mixer's output

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norms: Mapping[str, Norm]):
        if getattr(mixer, "has_output_bias", False) and not self.adds_output_bias:
            raise ValueError(f"{type(self).__name__} does not add the bias of its mixer's output projection")
        if set(norms) != set(self.NORMS):
            raise ValueError(
                f"{type(self).__name__} wants the norms {sorted(self.NORMS)}, the layer names {sorted(norms)}"
            )
        self.mixer, self.feed_forward = mixer, feed_forward
        self.norms = dict(norms)

    @property
    def mixer_norm(self) -> Norm:
        return self.norms["mixer"]

    @property
    def feed_forward_norm(self) -> Norm:
        return self.norms["feed_forward"]

    def parts(self) -> list[Part]:
        whole = [self.mixer, self.feed_forward, *(self.norms[name] for name in self.NORMS)]
        return [part for part in whole if part is not None]  # a layer may have no feed-forward

    def weight_specs(self) -> list[WeightSpec]:
        return [spec for part in self.parts() for spec in part.weight_specs()]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for part in self.parts():
            part.load(tensors)

    def forward(self, state: Residual, ctx: StepContext, cache: LayerCache) -> None:
        raise NotImplementedError


# ------------------------------------------------------------------------------ registries

Factory = Callable[..., Any]

MIXERS: dict[str, Factory] = {}
FEED_FORWARDS: dict[str, Factory] = {}
NORMS: dict[str, Factory] = {}
POSITION_ENCODINGS: dict[str, Factory] = {}
BLOCKS: dict[str, Factory] = {}
EMBEDDINGS: dict[str, Factory] = {}
HEADS: dict[str, Factory] = {}

_REGISTRIES = {
    "mixer": MIXERS,
    "feed_forward": FEED_FORWARDS,
    "norm": NORMS,
    "position_encoding": POSITION_ENCODINGS,
    "block": BLOCKS,
    "embedding": EMBEDDINGS,
    "head": HEADS,
}


def register(kind: str, name: str, replace: bool = False) -> Callable[[Factory], Factory]:
    """Class decorator: ``@register("mixer", "gqa_attention")``.

    A mixer, feed-forward, norm or position encoding is built as ``cls(prefix, hidden_size,
    **PartSpec.params)`` where ``prefix`` is the checkpoint prefix of the layer; a block as
    ``cls(mixer, feed_forward, norms)`` with ``norms`` a mapping from the names in its ``NORMS``
    to norm parts; an embedding or a head as ``cls(vocab_size, hidden_size, **PartSpec.params)``.
    """
    registry = _REGISTRIES[kind]

    def decorate(cls: Factory) -> Factory:
        if name in registry and not replace:
            raise ValueError(f"{kind} {name!r} is already registered")
        registry[name] = cls
        return cls

    return decorate


def build_end(kind: str, spec: PartSpec, vocab_size: int, hidden_size: int) -> Any:
    """An ``"embedding"`` or a ``"head"``: ``cls(vocab_size, hidden_size, **PartSpec.params)``."""
    registry = _REGISTRIES[kind]
    if spec.kind not in registry:
        raise KeyError(f"no {kind} named {spec.kind!r}; registered: {', '.join(sorted(registry))}")
    return registry[spec.kind](vocab_size, hidden_size, **dict(spec.params))


def build_part(kind: str, spec: PartSpec, prefix: str, hidden_size: int) -> Any:
    registry = _REGISTRIES[kind]
    if spec.kind not in registry:
        raise KeyError(f"no {kind} named {spec.kind!r}; registered: {', '.join(sorted(registry))}")
    return registry[spec.kind](prefix, hidden_size, **dict(spec.params))
