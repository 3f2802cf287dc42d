"""Typed configuration of the Daborax decoder, read from its own config.json keys.

config.json gives ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``residual_mult`` and a list ``layers``.  A
layer names its mixer ``type`` ("mamba2", "lightning" or "attention"), the mixer's sizes and constants under ``mixer``,
its feed-forward under ``mlp`` (null: none; ``kind`` "dense" with ``ff`` and ``limit``), and optionally ``weights_of``:
the layer whose tensors it runs with (it then has none of its own, but a cache or state of its own).  Every size and
constant of a model comes from this object.
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


def _number(d: dict, key: str, where: str, default=None) -> float:
    v = d.get(key, default)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v):
        raise ConfigError(f"{where}.{key} must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class StateSpaceConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    taps: int

    @staticmethod
    def from_dict(d: dict, where: str) -> "StateSpaceConfig":
        c = StateSpaceConfig(_pos_int(d, "heads", where), _pos_int(d, "vdim", where), _pos_int(d, "state", where),
                             _pos_int(d, "groups", where) if "groups" in d else 1,
                             _pos_int(d, "norm_groups", where) if "norm_groups" in d else 1, _pos_int(d, "conv", where))
        if c.heads % c.groups:
            raise ConfigError(f"{where}: {c.heads} heads do not divide into {c.groups} groups")
        if (c.heads * c.vdim) % c.norm_groups:
            raise ConfigError(f"{where}: {c.heads * c.vdim} inner values do not divide into {c.norm_groups} norm groups")
        return c


@dataclass(frozen=True)
class LinearAttentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]

    @staticmethod
    def from_dict(d: dict, where: str) -> "LinearAttentionConfig":
        heads = _pos_int(d, "heads", where)
        decay = d.get("decay")
        if isinstance(decay, (int, float)) and not isinstance(decay, bool):
            decay = [decay] * heads
        if not isinstance(decay, list) or len(decay) != heads or not all(
                isinstance(x, (int, float)) and not isinstance(x, bool) and math.isfinite(x) for x in decay):
            raise ConfigError(f"{where}.decay must list one number a head ({heads}), got {decay!r}")
        return LinearAttentionConfig(heads, _pos_int(d, "dim", where), _pos_int(d, "vdim", where),
                                     tuple(float(x) for x in decay))


@dataclass(frozen=True)
class SinkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float | None
    window: int | None

    @staticmethod
    def from_dict(d: dict, where: str) -> "SinkAttentionConfig":
        heads = _pos_int(d, "heads", where)
        kv_heads = _pos_int(d, "kv_heads", where) if "kv_heads" in d else heads
        if heads % kv_heads:
            raise ConfigError(f"{where}: {heads} heads are no multiple of {kv_heads} kv_heads")
        dim = _pos_int(d, "dim", where)
        window = (d.get("mask") or {}).get("size")
        if window is not None and (not isinstance(window, int) or isinstance(window, bool) or window <= 0):
            raise ConfigError(f"{where}.mask.size must be a positive integer, got {window!r}")
        cap = d.get("softcap")
        if cap is not None:
            cap = _number(d, "softcap", where)
            if cap <= 0:
                raise ConfigError(f"{where}.softcap must be positive, got {cap!r}")
        return SinkAttentionConfig(heads, kv_heads, dim, _pos_int(d, "vdim", where) if "vdim" in d else dim,
                                   _number(d, "scale", where, 1.0 / math.sqrt(dim)), cap, window)


@dataclass(frozen=True)
class ClampedFeedForwardConfig:
    ff: int
    limit: float

    @staticmethod
    def from_dict(d: dict | None, where: str) -> "ClampedFeedForwardConfig | None":
        if d is None:
            return None
        if d.get("kind") != "dense":
            raise ConfigError(f"{where}.kind={d.get('kind')!r} is not known ('dense')")
        limit = _number(d, "limit", where)
        if limit <= 0:
            raise ConfigError(f"{where}.limit must be positive, got {limit!r}")
        return ClampedFeedForwardConfig(_pos_int(d, "ff", where), limit)


_MIXERS = {"mamba2": StateSpaceConfig, "lightning": LinearAttentionConfig, "attention": SinkAttentionConfig}


@dataclass(frozen=True)
class DaboraxLayerConfig:
    type: str
    mixer: StateSpaceConfig | LinearAttentionConfig | SinkAttentionConfig
    mlp: ClampedFeedForwardConfig | None
    weights_of: int | None = None


@dataclass(frozen=True)
class DaboraxConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    residual_mult: float
    layers: tuple[DaboraxLayerConfig, ...]
    eos_token_id: tuple[int, ...] = ()

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @staticmethod
    def from_dict(d: dict[str, Any]) -> "DaboraxConfig":
        for key in ("vocab", "width", "layers"):
            if key not in d:
                raise ConfigError(f"config.json lacks the key {key!r}")
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers: list[DaboraxLayerConfig] = []
        for i, ld in enumerate(d["layers"]):
            where = f"layers[{i}]"
            kind = ld.get("type")
            if kind not in _MIXERS:
                raise ConfigError(f"{where}.type={kind!r} is not known ({', '.join(repr(k) for k in _MIXERS)})")
            layer = DaboraxLayerConfig(kind, _MIXERS[kind].from_dict(ld.get("mixer") or {}, where + ".mixer"),
                                       ClampedFeedForwardConfig.from_dict(ld.get("mlp"), where + ".mlp"), ld.get("weights_of"))
            j = layer.weights_of
            if j is not None:
                if not isinstance(j, int) or isinstance(j, bool) or not 0 <= j < i:
                    raise ConfigError(f"{where}.weights_of={j!r} must name an earlier layer")
                if layers[j].weights_of is not None:  # a layer that itself borrows: the tensors are its lender's
                    j = layers[j].weights_of
                    layer = DaboraxLayerConfig(layer.type, layer.mixer, layer.mlp, j)
                if layers[j].type != layer.type or (layers[j].mlp is None) != (layer.mlp is None):
                    raise ConfigError(f"{where}.weights_of={j}: layer {j} has another mixer type or feed-forward")
            layers.append(layer)
        eps = float((d.get("norm") or {}).get("eps", 1e-6))
        if not (eps > 0 and math.isfinite(eps)):
            raise ConfigError(f"norm.eps must be positive and finite, got {eps!r}")
        eos = d.get("eos_token_id")
        eos_t = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(int(e) for e in eos))
        return DaboraxConfig(
            vocab=_pos_int(d, "vocab", "config"), width=_pos_int(d, "width", "config"), norm_eps=eps,
            embedding_scale=_number(d.get("embedding") or {}, "scale", "embedding", 1.0),
            residual_mult=_number(d, "residual_mult", "config", 1.0), layers=tuple(layers), eos_token_id=eos_t)
