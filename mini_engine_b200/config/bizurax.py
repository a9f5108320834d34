"""Typed configuration of the Bizurax decoder, read from its own ``config.json`` keys.

``config.json`` gives ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``residual_mult`` (what every sublayer's
output is multiplied by before it enters the residual; absent: 1), ``streams`` (the number of residual streams of the
hyper-connections; absent or ``null``: one plain residual), ``loop`` (``start``, ``stop``, ``times``: layers ``start ..
stop - 1`` run ``times`` times in a row with the same weights, each pass with a cache of its own; absent: no layer
repeats) and ``layers``: one entry per layer with its ``type`` (``attention``, ``latent_attention`` or ``retention``),
the mixer's sizes and constants under ``mixer`` and its feed-forward under ``mlp`` (``null``: the layer has none;
``kind`` ``dense`` or ``moe``).  Layers may differ from one another in every size and come in any order.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from mini_engine_b200.config.pimezen import _need
from mini_engine_b200.config.qwen3 import ConfigError

NUMBER = (int, float)


@dataclass(frozen=True)
class Rotation:
    """Rotary positions on the first ``dims`` elements of a head; every frequency is divided by ``factor``."""

    base: float
    dims: int
    factor: float = 1.0

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str, most: int) -> "Rotation":
        scaling = raw.get("scaling")
        factor = 1.0 if scaling is None else float(_need(scaling, "factor", NUMBER, where + "scaling."))
        out = cls(base=float(_need(raw, "base", NUMBER, where)), dims=_need(raw, "dims", int, where), factor=factor)
        if out.dims % 2 or not 2 <= out.dims <= most:
            raise ConfigError(f"{where}dims must be even and between 2 and {most}, got {out.dims}")
        if not out.base > 0 or not out.factor > 0:
            raise ConfigError(f"{where}base and scaling.factor must be positive")
        return out

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.factor != 1.0:
            out["scaling"] = {"factor": self.factor}
        return out


@dataclass(frozen=True)
class SinkAttentionMixer:
    """Grouped-query attention with biased projections, unit q and k behind the rotation, capped scores and a sink."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float | None
    rot: Rotation

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "SinkAttentionMixer":
        cap = raw.get("softcap")
        if cap is not None and (isinstance(cap, bool) or not isinstance(cap, NUMBER) or not cap > 0):
            raise ConfigError(f"config.json key {where}'softcap' must be a positive number or absent, got {cap!r}")
        dim = _need(raw, "dim", int, where)
        out = cls(
            heads=_need(raw, "heads", int, where),
            kv_heads=_need(raw, "kv_heads", int, where),
            dim=dim,
            vdim=_need(raw, "vdim", int, where),
            scale=float(_need(raw, "scale", NUMBER, where)),
            softcap=None if cap is None else float(cap),
            rot=Rotation.from_dict(_need(raw, "rot", Mapping, where), where + "rot.", max(dim, 2)),
        )
        if min(out.heads, out.kv_heads, out.dim, out.vdim) < 1:
            raise ConfigError(f"{where}: sizes must be positive")
        if out.heads % out.kv_heads:
            raise ConfigError(f"{where}heads ({out.heads}) must be a multiple of kv_heads ({out.kv_heads})")
        return out

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                               "scale": self.scale, "rot": self.rot.to_dict()}  # fmt: skip
        if self.softcap is not None:
            out["softcap"] = self.softcap
        return out


@dataclass(frozen=True)
class DirectLatentAttentionMixer:
    """Attention whose keys and values are expanded from one cached latent per token; queries are projected directly."""

    heads: int
    dim: int  # plain query/key elements of a head
    rot_dim: int  # rotated ones
    vdim: int
    kv_rank: int
    scale: float
    rot: Rotation

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "DirectLatentAttentionMixer":
        rot_dim = _need(raw, "rot_dim", int, where)
        out = cls(
            heads=_need(raw, "heads", int, where),
            dim=_need(raw, "dim", int, where),
            rot_dim=rot_dim,
            vdim=_need(raw, "vdim", int, where),
            kv_rank=_need(raw, "kv_rank", int, where),
            scale=float(_need(raw, "scale", NUMBER, where)),
            rot=Rotation.from_dict(_need(raw, "rot", Mapping, where), where + "rot.", max(rot_dim, 2)),
        )
        if min(out.heads, out.dim, out.rot_dim, out.vdim, out.kv_rank) < 1:
            raise ConfigError(f"{where}: sizes must be positive")
        return out

    def to_dict(self) -> dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
                "scale": self.scale, "rot": self.rot.to_dict()}  # fmt: skip


@dataclass(frozen=True)
class RetentionMixer:
    """Linear attention with a fixed decay per head and a matrix state per head."""

    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]
    rot: Rotation

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "RetentionMixer":
        dim = _need(raw, "dim", int, where)
        decay = _need(raw, "decay", list, where)
        if not all(isinstance(a, NUMBER) and not isinstance(a, bool) for a in decay):
            raise ConfigError(f"{where}decay must be a list of numbers")
        out = cls(
            heads=_need(raw, "heads", int, where),
            dim=dim,
            vdim=_need(raw, "vdim", int, where),
            decay=tuple(float(a) for a in decay),
            rot=Rotation.from_dict(_need(raw, "rot", Mapping, where), where + "rot.", max(dim, 2)),
        )
        if min(out.heads, out.dim, out.vdim) < 1:
            raise ConfigError(f"{where}: sizes must be positive")
        if len(out.decay) != out.heads or not all(0.0 < a <= 1.0 for a in out.decay):
            raise ConfigError(f"{where}decay must hold one number in (0, 1] per head ({out.heads}), got {list(out.decay)}")
        return out

    def to_dict(self) -> dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay), "rot": self.rot.to_dict()}


@dataclass(frozen=True)
class FeedForward:
    """``dense``: ``ff`` features behind a squared relu.  ``moe``: ``experts`` gated units of ``ff`` features of which a
    token uses ``top``, and a gated unit of ``shared_ff`` features (0: none) that every token uses."""

    kind: str
    ff: int
    experts: int = 0
    top: int = 0
    shared_ff: int = 0

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "FeedForward":
        kind = _need(raw, "kind", str, where)
        if kind == "dense":
            out = cls("dense", _need(raw, "ff", int, where))
        elif kind == "moe":
            router = _need(raw, "router", Mapping, where)
            shared = raw.get("shared")
            out = cls(
                "moe",
                _need(_need(raw, "expert", Mapping, where), "ff", int, where + "expert."),
                experts=_need(router, "experts", int, where + "router."),
                top=_need(router, "top", int, where + "router."),
                shared_ff=0 if shared is None else _need(shared, "ff", int, where + "shared."),
            )
            if not 1 <= out.top <= out.experts or out.shared_ff < 0:
                raise ConfigError(f"{where}: 1 <= router.top <= router.experts, got {out.top} of {out.experts}")
        else:
            raise ConfigError(f"{where}kind {kind!r} is not a feed-forward of this design (known: 'dense', 'moe')")
        if out.ff < 1:
            raise ConfigError(f"{where}ff must be positive")
        return out

    def to_dict(self) -> dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        out: dict[str, Any] = {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff}
        return out


MIXERS = {"attention": SinkAttentionMixer, "latent_attention": DirectLatentAttentionMixer, "retention": RetentionMixer}


@dataclass(frozen=True)
class BizuraxLayer:
    type: str  # a key of MIXERS
    mixer: SinkAttentionMixer | DirectLatentAttentionMixer | RetentionMixer
    mlp: FeedForward | None

    def to_dict(self) -> dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class LayerLoop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class BizuraxConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    streams: int | None
    loop: LayerLoop | None
    layers: tuple[BizuraxLayer, ...]
    eos_token_ids: tuple[int, ...] = ()

    architecture = "Bizurax"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    def layer_order(self) -> list[int]:
        """The layers' numbers in the order they run: a loop's span repeated in place."""
        count = len(self.layers)
        if self.loop is None:
            return list(range(count))
        span = list(range(self.loop.start, self.loop.stop))
        return list(range(self.loop.start)) + span * self.loop.times + list(range(self.loop.stop, count))

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "BizuraxConfig":
        if raw.get("architecture") != cls.architecture:
            raise ConfigError(f"architecture must be {cls.architecture!r}, got {raw.get('architecture')!r}")
        norm = _need(raw, "norm", Mapping, "")
        layers: list[BizuraxLayer] = []
        for index, entry in enumerate(_need(raw, "layers", list, "")):
            where = f"layers[{index}]."
            kind = _need(entry, "type", str, where)
            if kind not in MIXERS:
                raise ConfigError(f"{where}type {kind!r} is not a mixer of this design (known: {', '.join(map(repr, MIXERS))})")
            mixer = MIXERS[kind].from_dict(_need(entry, "mixer", Mapping, where), where + "mixer.")
            mlp_raw = entry.get("mlp")
            layers.append(BizuraxLayer(kind, mixer, None if mlp_raw is None else FeedForward.from_dict(mlp_raw, where + "mlp.")))
        if not layers:
            raise ConfigError("config.json lists no layers")
        loop_raw, loop = raw.get("loop"), None
        if loop_raw is not None:
            loop = LayerLoop(*(_need(loop_raw, key, int, "loop.") for key in ("start", "stop", "times")))
            if not 0 <= loop.start < loop.stop <= len(layers) or loop.times < 1:
                raise ConfigError(f"loop must name layers start < stop <= {len(layers)} and times >= 1, got {loop}")
        streams = raw.get("streams")
        if streams is not None and (isinstance(streams, bool) or not isinstance(streams, int) or not 1 <= streams <= 8):
            raise ConfigError(f"config.json key 'streams' must be a number from 1 to 8 or absent, got {streams!r}")
        mult = raw.get("residual_mult")
        if mult is not None and (isinstance(mult, bool) or not isinstance(mult, NUMBER)):
            raise ConfigError(f"config.json key 'residual_mult' must be a number or absent, got {mult!r}")
        eos = raw.get("eos_token_id")
        out = cls(
            vocab=_need(raw, "vocab", int, ""),
            width=_need(raw, "width", int, ""),
            norm_eps=float(_need(norm, "eps", NUMBER, "norm.")),
            residual_mult=1.0 if mult is None else float(mult),
            streams=streams,
            loop=loop,
            layers=tuple(layers),
            eos_token_ids=() if eos is None else ((eos,) if isinstance(eos, int) else tuple(int(e) for e in eos)),
        )
        if out.vocab < 1 or out.width < 1 or not out.norm_eps > 0:
            raise ConfigError("vocab, width and norm.eps must be positive")
        return out

    @classmethod
    def from_folder(cls, folder: str | Path) -> "BizuraxConfig":
        return cls.from_dict(json.loads((Path(folder) / "config.json").read_text()))

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
            "residual_mult": self.residual_mult, "layers": [layer.to_dict() for layer in self.layers],
        }  # fmt: skip
        if self.streams is not None:
            out["streams"] = self.streams
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
