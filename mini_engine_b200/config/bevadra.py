"""Typed configuration of the Bevadra decoder, read from its own ``config.json`` keys.

``config.json`` gives ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``logit_softcap`` (absent or ``null``: the
logits are not capped) and ``layers``: one entry per layer with its ``type`` (``attention`` or ``latent_attention``),
the mixer's sizes and constants under ``mixer`` and its feed-forward under ``mlp`` (``null``: the layer has none).
Layers may differ from one another in every size and come in any order.  An attention layer with ``kv_from: j`` has
no keys and values of its own and reads layer ``j``'s.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from mini_engine_b200.config.pimezen import _need
from mini_engine_b200.config.qwen3 import ConfigError

NUMBER = (int, float)


def _window(raw: Mapping[str, Any], where: str) -> int | None:
    mask = raw.get("mask")
    window = None if mask is None else _need(mask, "size", int, where + "mask.")
    if window is not None and window < 1:
        raise ConfigError(f"{where}mask.size must be positive, got {window}")
    return window


@dataclass(frozen=True)
class BiasedAttentionMixer:
    """Grouped-query attention with a linear distance bias, a learned sink and a gate per element."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int | None  # mask.size: position i sees j when 0 <= i - j < window
    kv_from: int | None = None

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "BiasedAttentionMixer":
        kv_from = raw.get("kv_from")
        if kv_from is not None and (isinstance(kv_from, bool) or not isinstance(kv_from, int)):
            raise ConfigError(f"config.json key {where}'kv_from' must be a layer's number, got {kv_from!r}")
        out = cls(
            heads=_need(raw, "heads", int, where),
            kv_heads=_need(raw, "kv_heads", int, where),
            dim=_need(raw, "dim", int, where),
            vdim=_need(raw, "vdim", int, where),
            scale=float(_need(raw, "scale", NUMBER, where)),
            window=_window(raw, where),
            kv_from=kv_from,
        )
        if min(out.heads, out.kv_heads, out.dim, out.vdim) < 1:
            raise ConfigError(f"{where}: sizes must be positive")
        if out.heads % out.kv_heads:
            raise ConfigError(f"{where}heads ({out.heads}) must be a multiple of kv_heads ({out.kv_heads})")
        return out

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class LatentAttentionMixer:
    """Attention whose keys and values are expanded from one cached latent per token."""

    heads: int
    dim: int  # plain query/key elements of a head
    rot_dim: int  # rotated ones
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    window: int | None
    rot_base: float
    rot_dims: int  # how many of the rot_dim elements are rotated

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "LatentAttentionMixer":
        rot = _need(raw, "rot", Mapping, where)
        out = cls(
            heads=_need(raw, "heads", int, where),
            dim=_need(raw, "dim", int, where),
            rot_dim=_need(raw, "rot_dim", int, where),
            vdim=_need(raw, "vdim", int, where),
            kv_rank=_need(raw, "kv_rank", int, where),
            q_rank=_need(raw, "q_rank", int, where),
            scale=float(_need(raw, "scale", NUMBER, where)),
            window=_window(raw, where),
            rot_base=float(_need(rot, "base", NUMBER, where + "rot.")),
            rot_dims=_need(rot, "dims", int, where + "rot."),
        )
        if min(out.heads, out.dim, out.rot_dim, out.vdim, out.kv_rank, out.q_rank) < 1:
            raise ConfigError(f"{where}: sizes must be positive")
        if out.rot_dims % 2 or not 2 <= out.rot_dims <= out.rot_dim:
            raise ConfigError(f"{where}rot.dims must be even and at most rot_dim ({out.rot_dim}), got {out.rot_dims}")
        return out

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
            "q_rank": self.q_rank, "scale": self.scale, "rot": {"base": self.rot_base, "dims": self.rot_dims},
        }  # fmt: skip
        if self.window is not None:
            out["mask"] = {"size": self.window}
        return out


@dataclass(frozen=True)
class DenseFeedForward:
    ff: int

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "DenseFeedForward":
        if _need(raw, "kind", str, where) != "dense":
            raise ConfigError(f"{where}kind {raw['kind']!r} is not a feed-forward of this design (known: 'dense')")
        out = cls(ff=_need(raw, "ff", int, where))
        if out.ff < 1:
            raise ConfigError(f"{where}ff must be positive")
        return out

    def to_dict(self) -> dict[str, Any]:
        return {"kind": "dense", "ff": self.ff}


@dataclass(frozen=True)
class BevadraLayer:
    type: str  # "attention" or "latent_attention"
    mixer: BiasedAttentionMixer | LatentAttentionMixer
    mlp: DenseFeedForward | None

    def to_dict(self) -> dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class BevadraConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_softcap: float | None
    layers: tuple[BevadraLayer, ...]
    eos_token_ids: tuple[int, ...] = ()

    architecture = "Bevadra"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "BevadraConfig":
        if raw.get("architecture") != cls.architecture:
            raise ConfigError(f"architecture must be {cls.architecture!r}, got {raw.get('architecture')!r}")
        norm = _need(raw, "norm", Mapping, "")
        layers: list[BevadraLayer] = []
        for index, entry in enumerate(_need(raw, "layers", list, "")):
            where = f"layers[{index}]."
            kind = _need(entry, "type", str, where)
            mixer_raw = _need(entry, "mixer", Mapping, where)
            if kind == "attention":
                mixer: BiasedAttentionMixer | LatentAttentionMixer = BiasedAttentionMixer.from_dict(mixer_raw, where + "mixer.")
                source = mixer.kv_from
                if source is not None:
                    if not 0 <= source < index or layers[source].type != "attention" or layers[source].mixer.kv_from is not None:
                        raise ConfigError(f"{where}mixer.kv_from must name an earlier attention layer with keys and values of its own, got {source}")
                    owner = layers[source].mixer
                    if (owner.kv_heads, owner.dim, owner.vdim) != (mixer.kv_heads, mixer.dim, mixer.vdim):
                        raise ConfigError(f"{where}mixer: the key and value heads of layer {source} do not fit this layer's")
            elif kind == "latent_attention":
                mixer = LatentAttentionMixer.from_dict(mixer_raw, where + "mixer.")
            else:
                raise ConfigError(f"{where}type {kind!r} is not a mixer of this design (known: 'attention', 'latent_attention')")
            mlp_raw = entry.get("mlp")
            mlp = None if mlp_raw is None else DenseFeedForward.from_dict(mlp_raw, where + "mlp.")
            layers.append(BevadraLayer(kind, mixer, mlp))
        if not layers:
            raise ConfigError("config.json lists no layers")
        cap = raw.get("logit_softcap")
        if cap is not None and (isinstance(cap, bool) or not isinstance(cap, NUMBER) or not cap > 0):
            raise ConfigError(f"config.json key 'logit_softcap' must be a positive number or absent, got {cap!r}")
        eos = raw.get("eos_token_id")
        out = cls(
            vocab=_need(raw, "vocab", int, ""),
            width=_need(raw, "width", int, ""),
            norm_eps=float(_need(norm, "eps", NUMBER, "norm.")),
            logit_softcap=None if cap is None else float(cap),
            layers=tuple(layers),
            eos_token_ids=() if eos is None else ((eos,) if isinstance(eos, int) else tuple(int(e) for e in eos)),
        )
        if out.vocab < 1 or out.width < 1 or not out.norm_eps > 0:
            raise ConfigError("vocab, width and norm.eps must be positive")
        return out

    @classmethod
    def from_folder(cls, folder: str | Path) -> "BevadraConfig":
        return cls.from_dict(json.loads((Path(folder) / "config.json").read_text()))

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
            "layers": [layer.to_dict() for layer in self.layers],
        }  # fmt: skip
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
