"""Typed configuration of the Sozurax decoder, read from its own config.json keys.

config.json gives ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``canon.taps`` and a list ``layers``; each
layer names its mixer ``type`` ("hgrn2" or "latent_attention"), the mixer's sizes and constants under ``mixer``, and
its feed-forward under ``mlp`` (null: none; ``kind`` "dense" or "moe").  Every size of the model comes from this
object; nothing about a particular checkpoint is written down anywhere else.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any

from tokasaurus_b200.config.model_config import ConfigError


def _pos_int(d: dict, key: str, where: str) -> int:
    v = d.get(key)
    if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise ConfigError(f"{where}.{key} must be a positive integer, got {v!r}")
    return v


@dataclass(frozen=True)
class RecurrentMixerConfig:
    heads: int
    dim: int
    vdim: int

    @staticmethod
    def from_dict(d: dict, where: str) -> "RecurrentMixerConfig":
        return RecurrentMixerConfig(_pos_int(d, "heads", where), _pos_int(d, "dim", where), _pos_int(d, "vdim", where))


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int       # unrotated query/key values a head
    rot_dim: int   # rotated query/key values a head (the key's are shared by the heads)
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    window: int | None
    rot_base: float
    rot_dims: int
    kv_from: int | None = None

    @staticmethod
    def from_dict(d: dict, where: str) -> "LatentMixerConfig":
        rot = d.get("rot") or {}
        rot_dim = d.get("rot_dim", 0)
        if not isinstance(rot_dim, int) or rot_dim < 0:
            raise ConfigError(f"{where}.rot_dim must be a non-negative integer, got {rot_dim!r}")
        rot_dims = int(rot.get("dims", rot_dim))
        if rot_dims % 2 or rot_dims > rot_dim:
            raise ConfigError(f"{where}.rot.dims={rot_dims} must be even and at most rot_dim={rot_dim}")
        mask = d.get("mask") or {}
        window = mask.get("size")
        if window is not None and (not isinstance(window, int) or window <= 0):
            raise ConfigError(f"{where}.mask.size must be a positive integer, got {window!r}")
        dim = _pos_int(d, "dim", where)
        scale = d.get("scale")
        if scale is None:
            scale = 1.0 / math.sqrt(dim + rot_dim)
        kv_from = d.get("kv_from")
        if kv_from is not None and (not isinstance(kv_from, int) or kv_from < 0):
            raise ConfigError(f"{where}.kv_from must name a layer, got {kv_from!r}")
        return LatentMixerConfig(
            heads=_pos_int(d, "heads", where), dim=dim, rot_dim=rot_dim, vdim=_pos_int(d, "vdim", where),
            kv_rank=_pos_int(d, "kv_rank", where), q_rank=_pos_int(d, "q_rank", where), scale=float(scale),
            window=window, rot_base=float(rot.get("base", 10000.0)), rot_dims=rot_dims, kv_from=kv_from)


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                 # "dense" or "moe"
    ff: int                   # inner size (of one expert for "moe")
    experts: int = 0
    top: int = 0
    shared_ff: int | None = None

    @staticmethod
    def from_dict(d: dict | None, where: str) -> "FeedForwardConfig | None":
        if d is None:
            return None
        kind = d.get("kind")
        if kind == "dense":
            return FeedForwardConfig("dense", _pos_int(d, "ff", where))
        if kind == "moe":
            router = d.get("router") or {}
            experts, top = _pos_int(router, "experts", where + ".router"), _pos_int(router, "top", where + ".router")
            if top > experts:
                raise ConfigError(f"{where}.router.top={top} exceeds experts={experts}")
            shared = d.get("shared")
            return FeedForwardConfig("moe", _pos_int(d.get("expert") or {}, "ff", where + ".expert"), experts, top,
                                     _pos_int(shared, "ff", where + ".shared") if shared is not None else None)
        raise ConfigError(f"{where}.kind={kind!r} is not known ('dense', 'moe')")


@dataclass(frozen=True)
class SozuraxLayerConfig:
    type: str
    mixer: RecurrentMixerConfig | LatentMixerConfig
    mlp: FeedForwardConfig | None


@dataclass(frozen=True)
class SozuraxConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    taps: int
    layers: tuple[SozuraxLayerConfig, ...]
    eos_token_id: tuple[int, ...] = ()

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @staticmethod
    def from_dict(d: dict[str, Any]) -> "SozuraxConfig":
        for key in ("vocab", "width", "layers"):
            if key not in d:
                raise ConfigError(f"config.json lacks the key {key!r}")
        layers = []
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        for i, ld in enumerate(d["layers"]):
            where = f"layers[{i}]"
            kind = ld.get("type")
            if kind == "hgrn2":
                mixer = RecurrentMixerConfig.from_dict(ld.get("mixer") or {}, where + ".mixer")
            elif kind == "latent_attention":
                mixer = LatentMixerConfig.from_dict(ld.get("mixer") or {}, where + ".mixer")
            else:
                raise ConfigError(f"{where}.type={kind!r} is not known ('hgrn2', 'latent_attention')")
            layers.append(SozuraxLayerConfig(kind, mixer, FeedForwardConfig.from_dict(ld.get("mlp"), where + ".mlp")))
        for i, layer in enumerate(layers):
            m = layer.mixer
            if isinstance(m, LatentMixerConfig) and m.kv_from is not None:
                src = layers[m.kv_from].mixer if m.kv_from < i else None
                if not isinstance(src, LatentMixerConfig) or src.kv_from is not None:
                    raise ConfigError(f"layers[{i}].mixer.kv_from={m.kv_from} must name an earlier latent-attention layer "
                                      "that makes its own latent")
                if (src.kv_rank, src.rot_dim, src.rot_base, src.rot_dims) != (m.kv_rank, m.rot_dim, m.rot_base, m.rot_dims):
                    raise ConfigError(f"layers[{i}] reads layer {m.kv_from}'s latent but differs in kv_rank, rot_dim or rotation")
        eps = float((d.get("norm") or {}).get("eps", 1e-6))
        if not (eps > 0 and math.isfinite(eps)):
            raise ConfigError(f"norm.eps must be positive and finite, got {eps!r}")
        eos = d.get("eos_token_id")
        eos_t = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(int(e) for e in eos))
        return SozuraxConfig(
            vocab=_pos_int(d, "vocab", "config"), width=_pos_int(d, "width", "config"), norm_eps=eps,
            embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)),
            taps=int((d.get("canon") or {}).get("taps", 1)), layers=tuple(layers), eos_token_id=eos_t)
