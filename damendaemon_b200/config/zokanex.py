"""Typed Zokanex configuration, parsed from the architecture's own config.json keys.

    architecture   "Zokanex"
    vocab, width   sizes of the token table and the residual stream
    embedding      {scale}: multiplies the token's row
    norm           {eps}: of every RMS norm (the layers', the heads' and the final one)
    layers         a list; each entry {type: "attention" | "retention", mixer: {...}, mlp: {...} | null}
      attention    {heads, kv_heads, dim, vdim, scale, rot: {dims, base} | absent, mask: {size} | absent,
                    kv_from: j (optional: no key/value tensors of its own, reads layer j's cache)}
      retention    {heads, dim, vdim, decay: [one per head], rot: {dims, base} | absent}
      mlp          {kind: "dense", ff} | {kind: "moe", router: {experts, top, scale, groups: {count, keep} | absent},
                    expert: {ff}, shared: {ff} | absent}

The configuration names no context length: the engine's cache sets it.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

from .reader import ConfigError

ARCHITECTURE = "Zokanex"


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
class Rotary:
    dims: int
    base: float


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[Rotary] = None
    mask_size: Optional[int] = None
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class RetentionMixer:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rot: Optional[Rotary] = None


@dataclass(frozen=True)
class Mlp:
    kind: str                       # 'dense' | 'moe'
    ff: int = 0                     # dense: the inner width; moe: an expert's
    experts: int = 0
    top: int = 0
    groups: int = 1
    keep: int = 1
    scale: float = 1.0
    shared_ff: Optional[int] = None


@dataclass(frozen=True)
class Layer:
    type: str                       # 'attention' | 'retention'
    mixer: object
    mlp: Optional[Mlp]


def _rotary(raw, dim, where):
    r = raw.get("rot")
    if r is None:
        return None
    dims = _positive_int(r, "dims", where + ".rot")
    if dims % 2 or dims > dim:
        raise ConfigError(f"{where}.rot.dims must be even and at most dim, got {dims}")
    base = _number(r, "base", where + ".rot")
    if base == 1.0:
        raise ConfigError(f"{where}.rot.base must not be 1")
    return Rotary(dims, base)


def _attention(raw, where):
    sizes = {n: _positive_int(raw, n, where) for n in ("heads", "kv_heads", "dim", "vdim")}
    if sizes["heads"] % sizes["kv_heads"]:
        raise ConfigError(f"{where}: {sizes['heads']} heads cannot share {sizes['kv_heads']} key/value heads")
    mask = raw.get("mask")
    source = raw.get("kv_from")
    if source is not None and (type(source) is not int or source < 0):
        raise ConfigError(f"{where}.kv_from must name a layer, got {source!r}")
    return AttentionMixer(scale=_number(raw, "scale", where), rot=_rotary(raw, sizes["dim"], where),
                          mask_size=None if mask is None else _positive_int(mask, "size", where + ".mask"),
                          kv_from=source, **sizes)


def _retention(raw, where):
    sizes = {n: _positive_int(raw, n, where) for n in ("heads", "dim", "vdim")}
    decay = _get(raw, "decay", where)
    if not isinstance(decay, list) or len(decay) != sizes["heads"] or \
            any(type(d) not in (int, float) or not math.isfinite(d) or not 0.0 <= d <= 1.0 for d in decay):
        raise ConfigError(f"{where}.decay must list one number in [0, 1] per head ({sizes['heads']}), got {decay!r}")
    return RetentionMixer(decay=tuple(float(d) for d in decay), rot=_rotary(raw, sizes["dim"], where), **sizes)


def _mlp(raw, where):
    if raw is None:
        return None
    kind = _get(raw, "kind", where)
    if kind == "dense":
        return Mlp("dense", ff=_positive_int(raw, "ff", where))
    if kind == "moe":
        router = _get(raw, "router", where)
        experts, top = _positive_int(router, "experts", where + ".router"), _positive_int(router, "top", where + ".router")
        groups, keep = 1, 1
        if router.get("groups") is not None:
            groups = _positive_int(router["groups"], "count", where + ".router.groups")
            keep = _positive_int(router["groups"], "keep", where + ".router.groups")
        if experts % groups or keep > groups:
            raise ConfigError(f"{where}.router: {experts} experts do not form {groups} equal groups of which {keep} stay")
        if top > experts // groups * keep:
            raise ConfigError(f"{where}.router: {top} experts per token, but only {experts // groups * keep} can be chosen")
        scale = _number(router, "scale", where + ".router") if "scale" in router else 1.0
        shared = raw.get("shared")
        return Mlp("moe", ff=_positive_int(_get(raw, "expert", where), "ff", where + ".expert"), experts=experts, top=top,
                   groups=groups, keep=keep, scale=scale,
                   shared_ff=None if shared is None else _positive_int(shared, "ff", where + ".shared"))
    raise ConfigError(f"{where}.kind must be 'dense' or 'moe', got {kind!r}")


@dataclass(frozen=True)
class ZokanexConfig:
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
    def from_dict(cls, config: dict) -> "ZokanexConfig":
        if config.get("architecture") != ARCHITECTURE:
            raise ConfigError(f"architecture must be {ARCHITECTURE!r}, got {config.get('architecture')!r}")
        raw_layers = _get(config, "layers", "config")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("layers must be a non-empty list")
        layers = []
        for i, raw in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = _get(raw, "type", where)
            if kind == "attention":
                mixer = _attention(_get(raw, "mixer", where), where + ".mixer")
                j = mixer.kv_from
                if j is not None:
                    if j >= i or layers[j].type != "attention" or layers[j].mixer.kv_from is not None:
                        raise ConfigError(f"{where}.mixer.kv_from must name an earlier attention layer with keys and values "
                                          f"of its own, got {j!r}")
                    theirs = layers[j].mixer
                    if (theirs.kv_heads, theirs.dim, theirs.vdim, theirs.rot) != (mixer.kv_heads, mixer.dim, mixer.vdim, mixer.rot):
                        raise ConfigError(f"{where}.mixer reads layer {j}'s keys and values but has other head sizes or another rotation")
            elif kind == "retention":
                mixer = _retention(_get(raw, "mixer", where), where + ".mixer")
            else:
                raise ConfigError(f"{where}.type must be 'attention' or 'retention', got {kind!r}")
            layers.append(Layer(kind, mixer, _mlp(raw.get("mlp"), where + ".mlp")))
        return cls(vocab=_positive_int(config, "vocab", "config"), width=_positive_int(config, "width", "config"),
                   embedding_scale=_number(_get(config, "embedding", "config"), "scale", "embedding"),
                   norm_eps=_number(_get(config, "norm", "config"), "eps", "norm"), layers=tuple(layers))

    def to_dict(self) -> dict:
        """The config.json this configuration round-trips through."""
        layers = []
        for layer in self.layers:
            m = layer.mixer
            mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim}
            if m.rot is not None:
                mixer["rot"] = {"dims": m.rot.dims, "base": m.rot.base}
            if layer.type == "attention":
                mixer.update(kv_heads=m.kv_heads, scale=m.scale)
                if m.mask_size is not None:
                    mixer["mask"] = {"size": m.mask_size}
                if m.kv_from is not None:
                    mixer["kv_from"] = m.kv_from
            else:
                mixer["decay"] = list(m.decay)
            mlp = None
            if layer.mlp is not None and layer.mlp.kind == "dense":
                mlp = {"kind": "dense", "ff": layer.mlp.ff}
            elif layer.mlp is not None:
                f = layer.mlp
                mlp = {"kind": "moe", "expert": {"ff": f.ff},
                       "router": {"experts": f.experts, "top": f.top, "scale": f.scale, "groups": {"count": f.groups, "keep": f.keep}}}
                if f.shared_ff is not None:
                    mlp["shared"] = {"ff": f.shared_ff}
            layers.append({"type": layer.type, "mixer": mixer, "mlp": mlp})
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps}, "layers": layers}
