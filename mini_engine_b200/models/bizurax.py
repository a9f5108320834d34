"""Bizurax laid out as parts.

Pre-norm layers (RMS norms) on several residual streams (hyper-connections: every sublayer reads a learned sum of the
streams, and its output, times a constant of the model, enters every stream with a learned share while a learned
matrix mixes the streams), or on one plain residual when the configuration names no streams.  A span of layers may
run several times in a row with the same weights; every pass keeps a cache or a state of its own.  A layer's mixer
is one of

* ``attention``: grouped-query attention with biases on q, k and v, a rotation (rotate-half, possibly on a part of the
  head, frequencies divided by a scaling factor), q and k divided by their root mean square per head *behind* the
  rotation, scores scaled and then capped by ``cap * tanh(s / cap)``, and a softmax whose denominator has one more
  term ``exp(sink_h)`` with a learned number per head;
* ``latent_attention``: queries projected directly, keys and values expanded from one cached normed latent per token
  plus one rotated key part that all heads share (pairs of neighbouring elements are rotated), an ordinary softmax;
* ``retention``: linear attention with a fixed decay per head, rotated q and k, a 32-bit matrix state per head, unit
  norm per head and a silu gate.

The feed-forward is a squared-relu unit without a gate, or routed gated units (a biased router in 32-bit, the ``top``
largest logits, softmax over the chosen ones) beside a shared gated unit.  The model ends in an RMS norm of the sum
of the streams and a head of its own.  Every size and every constant that models of this design may differ in comes
from the typed configuration, layer by layer.
"""

from __future__ import annotations

from mini_engine_b200.config.bizurax import (
    BizuraxConfig,
    DirectLatentAttentionMixer,
    FeedForward,
    RetentionMixer,
    Rotation,
    SinkAttentionMixer,
)
from mini_engine_b200.config.model_spec import LayerSpec, ModelSpec, OrderEntry, PartSpec
from mini_engine_b200.config.registry import Architecture, register_architecture


def _rope(rot: Rotation, head_dim: int) -> PartSpec:
    return PartSpec("rope", {"head_dim": head_dim, "theta": rot.base, "rotary_dim": rot.dims, "frequency_divisor": rot.factor})


def _attention(mixer: SinkAttentionMixer, eps: float) -> PartSpec:
    return PartSpec(
        "gqa_attention",
        {
            "num_heads": mixer.heads, "kv_heads": mixer.kv_heads, "head_dim": mixer.dim, "value_dim": mixer.vdim,
            "qk_norm_eps": None, "position_encoding": _rope(mixer.rot, mixer.dim), "scale": mixer.scale, "qkv_bias": True,
            "softmax_sink": "learned", "unit_norm_eps": eps, "score_softcap": mixer.softcap,
            "names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o", "q_bias": "mix.q.b", "k_bias": "mix.k.b",
                      "v_bias": "mix.v.b", "sink": "mix.sink"},
        },
    )  # fmt: skip


def _latent_attention(mixer: DirectLatentAttentionMixer, eps: float) -> PartSpec:
    return PartSpec(
        "latent_attention",
        {
            "num_heads": mixer.heads, "head_dim": mixer.dim, "rot_dim": mixer.rot_dim, "value_dim": mixer.vdim,
            "kv_rank": mixer.kv_rank, "q_rank": None, "norm_eps": eps, "scale": mixer.scale,
            "position_encoding": _rope(mixer.rot, mixer.rot_dim), "rotary_layout": "interleaved",
            "names": {"q": "mix.q", "dkv": "mix.dkv", "kv_norm": "mix.dkv.norm", "uk": "mix.uk", "uv": "mix.uv", "o": "mix.o"},
        },
    )  # fmt: skip


def _retention(mixer: RetentionMixer, eps: float) -> PartSpec:
    return PartSpec(
        "retention",
        {
            "num_heads": mixer.heads, "head_dim": mixer.dim, "value_dim": mixer.vdim, "decay": mixer.decay, "norm_eps": eps,
            "position_encoding": _rope(mixer.rot, mixer.dim),
            "names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "g": "mix.g", "o": "mix.o"},
        },
    )  # fmt: skip


def _feed_forward(mlp: FeedForward) -> PartSpec:
    if mlp.kind == "dense":
        return PartSpec("mlp", {"intermediate_size": mlp.ff, "activation": "relu_squared", "names": {"up": "mlp.up", "down": "mlp.down"}})
    return PartSpec(
        "routed_experts",
        {
            "units": mlp.experts, "top": mlp.top, "intermediate_size": mlp.ff, "router_bias": True, "scoring": "softmax_chosen",
            "shared_intermediate_size": mlp.shared_ff or None,
            "names": {"router": "mlp.router", "router_bias": "mlp.router.b", "unit": "mlp.e{index}.", "shared": "mlp.shared.",
                      "gate": "gate", "up": "up", "down": "down"},
        },
    )  # fmt: skip


_MIXERS = {"attention": _attention, "latent_attention": _latent_attention, "retention": _retention}


def bizurax_spec(cfg: BizuraxConfig) -> ModelSpec:
    eps = cfg.norm_eps
    layers = []
    for index, layer in enumerate(cfg.layers):
        norms = {"mixer_norm": PartSpec("rmsnorm", {"name": "norm1", "eps": eps})}
        subs = ("mixer",) if layer.mlp is None else ("mixer", "feed_forward")
        if layer.mlp is not None:
            norms["feed_forward_norm"] = PartSpec("rmsnorm", {"name": "norm2", "eps": eps})
        # a checkpoint may carry the second sublayer's norm and coefficients for a layer that has no feed-forward
        unused = () if layer.mlp is not None else ("norm2",) if cfg.streams is None else ("norm2", "hc2.in", "hc2.mix", "hc2.out")
        if cfg.streams is None:
            block, params = "prenorm", {"residual_mult": cfg.residual_mult, "unused_names": unused}
        else:
            tensors = {"mixer": "hc1", "feed_forward": "hc2"}
            names = {sub: {"read": tensors[sub] + ".in", "mix": tensors[sub] + ".mix", "share": tensors[sub] + ".out"} for sub in subs}
            block, params = "hyper_prenorm", {"streams": cfg.streams, "names": names, "residual_mult": cfg.residual_mult, "unused_names": unused}
        layers.append(
            LayerSpec(
                prefix=f"l{index}.", block=block + ("_mixer_only" if layer.mlp is None else ""),
                mixer=_MIXERS[layer.type](layer.mixer, eps),
                feed_forward=None if layer.mlp is None else _feed_forward(layer.mlp), block_params=params, **norms,
            )
        )  # fmt: skip
    return ModelSpec(
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        embedding=PartSpec("token_embedding", {"weight": "embed"}),
        layers=tuple(layers),
        order=tuple(OrderEntry(index) for index in cfg.layer_order()),
        final_norm=PartSpec("rmsnorm", {"name": "final.norm", "eps": eps}),
        head=PartSpec("linear_head", {"weight": "head"}),
    )


register_architecture(
    Architecture(
        name=BizuraxConfig.architecture,
        read_config=BizuraxConfig.from_folder,
        build_spec=bizurax_spec,
        config_type=BizuraxConfig,
    )
)
