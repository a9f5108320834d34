"""Bevadra laid out as parts.

Every layer is parallel: one layer norm (weight and bias), and the mixer and the feed-forward both read its output,
``x = x + (mixer(norm1(x)) + ff(norm1(x)))``.  A layer's mixer is one of

* ``attention``: grouped-query attention without rotation, with biases on the q, k, v and output projections; a
  distance bias ``slope_h * (i - j)`` with fixed slopes is taken off the scaled scores; a sliding window; a softmax
  whose denominator has one more term ``exp(sink_h)`` with a learned number per head; the concatenated heads are
  multiplied element by element with ``sigmoid(W_g h)``; a layer may read an earlier layer's keys and values
  instead of making its own;
* ``latent_attention``: queries through a normed latent, keys and values expanded from one cached normed latent per
  token plus one rotated key part that all heads share, a sliding window, an ordinary softmax and a sigmoid gate
  per head.

The feed-forward is a gated unit with the tanh form of GELU.  The model ends in a layer norm and the embedding
matrix as the head, with the logits soft-capped.  Every size and every constant that models of this design may
differ in comes from the typed configuration, layer by layer; the constants below are fixed by the design.
"""

from __future__ import annotations

from mini_engine_b200.config.bevadra import BevadraConfig, BiasedAttentionMixer, DenseFeedForward, LatentAttentionMixer
from mini_engine_b200.config.model_spec import LayerSpec, ModelSpec, OrderEntry, PartSpec
from mini_engine_b200.config.registry import Architecture, register_architecture

BIAS_SPAN = 8.0  # slope_h = 2 ** (-8 (h + 1) / heads)


def _attention(mixer: BiasedAttentionMixer) -> PartSpec:
    return PartSpec(
        "gqa_attention",
        {
            "num_heads": mixer.heads, "kv_heads": mixer.kv_heads, "head_dim": mixer.dim, "value_dim": mixer.vdim,
            "qk_norm_eps": None, "position_encoding": None, "window": mixer.window, "scale": mixer.scale,
            "qkv_bias": True, "o_bias": True, "distance_bias": "linear", "linear_bias_span": BIAS_SPAN,
            "softmax_sink": "learned", "element_gate": True, "reads_shared_cache": mixer.kv_from is not None,
            "names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o", "q_bias": "mix.q.b", "k_bias": "mix.k.b",
                      "v_bias": "mix.v.b", "o_bias": "mix.o.b", "gate": "mix.g", "sink": "mix.sink"},
        },
    )  # fmt: skip


def _latent_attention(mixer: LatentAttentionMixer, eps: float) -> PartSpec:
    return PartSpec(
        "latent_attention",
        {
            "num_heads": mixer.heads, "head_dim": mixer.dim, "rot_dim": mixer.rot_dim, "value_dim": mixer.vdim,
            "kv_rank": mixer.kv_rank, "q_rank": mixer.q_rank, "norm_eps": eps, "scale": mixer.scale, "window": mixer.window,
            "position_encoding": PartSpec("rope", {"head_dim": mixer.rot_dims, "theta": mixer.rot_base, "rotary_dim": mixer.rot_dims}),
            "head_gate": True,
            "names": {"dq": "mix.dq", "q_norm": "mix.dq.norm", "uq": "mix.uq", "dkv": "mix.dkv", "kv_norm": "mix.dkv.norm",
                      "uk": "mix.uk", "uv": "mix.uv", "gate": "mix.g", "o": "mix.o"},
        },
    )  # fmt: skip


def _feed_forward(mlp: DenseFeedForward) -> PartSpec:
    return PartSpec(
        "gated_mlp",
        {"intermediate_size": mlp.ff, "activation": "gelu_tanh", "names": {"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"}},
    )


def bevadra_spec(cfg: BevadraConfig) -> ModelSpec:
    eps = cfg.norm_eps
    layers, order = [], []
    for index, layer in enumerate(cfg.layers):
        mixer = _attention(layer.mixer) if layer.type == "attention" else _latent_attention(layer.mixer, eps)
        layers.append(
            LayerSpec(
                prefix=f"l{index}.", block="parallel", mixer=mixer,
                feed_forward=None if layer.mlp is None else _feed_forward(layer.mlp),
                mixer_norm=PartSpec("layernorm", {"name": "norm1", "eps": eps}),
            )
        )  # fmt: skip
        order.append(OrderEntry(index, cache_of=getattr(layer.mixer, "kv_from", None)))
    return ModelSpec(
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        embedding=PartSpec("token_embedding", {"weight": "embed"}),
        layers=tuple(layers),
        order=tuple(order),
        final_norm=PartSpec("layernorm", {"name": "final.norm", "eps": eps}),
        head=PartSpec("linear_head", {"weight": "head.tied", "tied_to": "embed", "soft_cap": cfg.logit_softcap}),
    )


register_architecture(
    Architecture(
        name=BevadraConfig.architecture,
        read_config=BevadraConfig.from_folder,
        build_spec=bevadra_spec,
        config_type=BevadraConfig,
    )
)
