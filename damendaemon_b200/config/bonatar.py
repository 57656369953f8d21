"""Typed Bonatar configuration, parsed from the architecture's own config.json keys.

    architecture   "Bonatar"
    vocab, width   sizes of the token table and the residual stream
    embedding      {scale}: multiplies the token's row
    norm           {eps}: of every RMS norm
    layers         a list; each entry {type: "attention", mixer: {...}, mlp: {...} | null, weights_of: j (optional)}
      mixer        {heads, kv_heads, dim, vdim, scale, rot: {dims, base, scaling: {factor, original, fast, slow} | null}
                    | null, mask: {size} | null}
      mlp          {kind: "dense", ff} | {kind: "moe", router: {experts, top}, expert: {ff, limit},
                    shared: {ff, limit} | absent}
      weights_of   the entry has no tensors of its own and runs layer j's (with a cache of its own)

The configuration names no context length: the engine's cache sets it.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

from .reader import ConfigError

ARCHITECTURE = "Bonatar"


def _get(config, name, where):
    if not isinstance(config, dict) or name not in config:
        raise ConfigError(f"{where}: '{name}' is missing")
    return config[name]


def _positive_int(config, name, where):
    value = _get(config, name, where)
    if type(value) is not int or value <= 0:
        raise ConfigError(f"{where}.{name} must be a positive integer, got {value!r}")
    return value


def _number(config, name, where, positive=True):
    value = _get(config, name, where)
    if type(value) not in (int, float) or not math.isfinite(value) or (positive and value <= 0):
        raise ConfigError(f"{where}.{name} must be a finite{' positive' if positive else ''} number, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class RotaryScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class Rotary:
    dims: int
    base: float
    scaling: Optional[RotaryScaling] = None


@dataclass(frozen=True)
class Mixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[Rotary] = None
    mask_size: Optional[int] = None


@dataclass(frozen=True)
class Unit:
    ff: int
    limit: float


@dataclass(frozen=True)
class Mlp:
    kind: str                       # 'dense' | 'moe'
    ff: int = 0                     # dense
    experts: int = 0                # moe
    top: int = 0
    expert: Optional[Unit] = None
    shared: Optional[Unit] = None


@dataclass(frozen=True)
class Layer:
    type: str
    mixer: Mixer
    mlp: Optional[Mlp]
    weights_of: Optional[int] = None


def _mixer(raw, where):
    sizes = {n: _positive_int(raw, n, where) for n in ("heads", "kv_heads", "dim", "vdim")}
    if sizes["heads"] % sizes["kv_heads"]:
        raise ConfigError(f"{where}: {sizes['heads']} heads cannot share {sizes['kv_heads']} key/value heads")
    rot = None
    if raw.get("rot") is not None:
        r = raw["rot"]
        dims = _positive_int(r, "dims", where + ".rot")
        if dims % 2 or dims > sizes["dim"]:
            raise ConfigError(f"{where}.rot.dims must be even and at most dim, got {dims}")
        scaling = None
        if r.get("scaling") is not None:
            scaling = RotaryScaling(**{n: _number(r["scaling"], n, where + ".rot.scaling")
                                       for n in ("factor", "original", "fast", "slow")})
        base = _number(r, "base", where + ".rot")
        if base == 1.0:
            raise ConfigError(f"{where}.rot.base must not be 1")
        rot = Rotary(dims, base, scaling)
    mask = raw.get("mask")
    mask_size = None if mask is None else _positive_int(mask, "size", where + ".mask")
    return Mixer(scale=_number(raw, "scale", where), rot=rot, mask_size=mask_size, **sizes)


def _unit(raw, where):
    return Unit(_positive_int(raw, "ff", where), _number(raw, "limit", where))


def _mlp(raw, where):
    if raw is None:
        return None
    kind = _get(raw, "kind", where)
    if kind == "dense":
        return Mlp("dense", ff=_positive_int(raw, "ff", where))
    if kind == "moe":
        router = _get(raw, "router", where)
        experts, top = _positive_int(router, "experts", where + ".router"), _positive_int(router, "top", where + ".router")
        if top > experts:
            raise ConfigError(f"{where}.router: {top} experts per token of {experts}")
        shared = raw.get("shared")
        return Mlp("moe", experts=experts, top=top, expert=_unit(_get(raw, "expert", where), where + ".expert"),
                   shared=None if shared is None else _unit(shared, where + ".shared"))
    raise ConfigError(f"{where}.kind must be 'dense' or 'moe', got {kind!r}")


@dataclass(frozen=True)
class BonatarConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[Layer, ...]
    eos_token_ids: tuple = ()

    architecture = ARCHITECTURE

    @property
    def vocab_size(self):
        return self.vocab

    @classmethod
    def from_dict(cls, config: dict) -> "BonatarConfig":
        if config.get("architecture") != ARCHITECTURE:
            raise ConfigError(f"architecture must be {ARCHITECTURE!r}, got {config.get('architecture')!r}")
        raw_layers = _get(config, "layers", "config")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("layers must be a non-empty list")
        layers = []
        for i, raw in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = _get(raw, "type", where)
            if kind != "attention":
                raise ConfigError(f"{where}.type must be 'attention', got {kind!r}")
            source = raw.get("weights_of")
            if source is not None:
                if type(source) is not int or not 0 <= source < i or layers[source].weights_of is not None:
                    raise ConfigError(f"{where}.weights_of must name an earlier layer with tensors of its own, got {source!r}")
            layer = Layer(kind, _mixer(_get(raw, "mixer", where), where + ".mixer"), _mlp(raw.get("mlp"), where + ".mlp"), source)
            if source is not None and (layer.mixer, layer.mlp) != (layers[source].mixer, layers[source].mlp):
                raise ConfigError(f"{where} runs layer {source}'s weights but describes another mixer or feed-forward")
            layers.append(layer)
        return cls(vocab=_positive_int(config, "vocab", "config"), width=_positive_int(config, "width", "config"),
                   embedding_scale=_number(_get(config, "embedding", "config"), "scale", "embedding"),
                   norm_eps=_number(_get(config, "norm", "config"), "eps", "norm"), layers=tuple(layers))

    def to_dict(self) -> dict:
        """The config.json this configuration round-trips through."""
        layers = []
        for layer in self.layers:
            m = layer.mixer
            mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                     "rot": None, "mask": None if m.mask_size is None else {"size": m.mask_size}}
            if m.rot is not None:
                s = m.rot.scaling
                mixer["rot"] = {"dims": m.rot.dims, "base": m.rot.base, "scaling": None if s is None else
                                {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}}
            mlp = None
            if layer.mlp is not None and layer.mlp.kind == "dense":
                mlp = {"kind": "dense", "ff": layer.mlp.ff}
            elif layer.mlp is not None:
                mlp = {"kind": "moe", "router": {"experts": layer.mlp.experts, "top": layer.mlp.top},
                       "expert": {"ff": layer.mlp.expert.ff, "limit": layer.mlp.expert.limit}}
                if layer.mlp.shared is not None:
                    mlp["shared"] = {"ff": layer.mlp.shared.ff, "limit": layer.mlp.shared.limit}
            entry = {"type": layer.type, "mixer": mixer, "mlp": mlp}
            if layer.weights_of is not None:
                entry["weights_of"] = layer.weights_of
            layers.append(entry)
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps}, "layers": layers}
