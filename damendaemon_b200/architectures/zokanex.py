"""Zokanex described with the framework's parts.

A decoder of parallel layers over a float32 stream that starts as the token's row times a scale: one RMS norm a
layer, whose output both the mixer and the feed-forward read, and both results are added to the stream. A mixer is
either grouped-query softmax attention (separate key and value head sizes; an RMS norm over every query head and
every key head, one weight per kind, before the rotation; rotary positions on the first dimensions of a head, the two
halves of the rotated stretch paired; a sliding window; a layer may have no keys and values of its own and read an
earlier layer's cache with its own queries and mask) or retention (a decaying outer-product state per head and
request in float32, rotated queries and keys, the read-out divided by its root mean square per head, a silu gate).
A feed-forward is one gated unit (tanh-gelu), or experts (silu units) chosen by sigmoid router scores within the
worthiest groups of neighbours, weighted by their scores, with a shared unit behind a sigmoid gate, or absent. The
final norm and an untied head give the logits.

Tensor names: embed, l<i>.norm1, l<i>.mix.{q,k,v,o,q.norm,k.norm} (attention) or l<i>.mix.{q,k,v,g,o} (retention),
l<i>.mlp.{gate,up,down} or l<i>.mlp.{router, e<j>.{gate,up,down}, shared.{gate,up,down,sg}}, final.norm, head;
matrices [out, in].
"""
from __future__ import annotations

import math

import torch

from ..config.zokanex import ARCHITECTURE, ZokanexConfig
from ..parts.spec import (AttentionSpec, EmbeddingSpec, GatedFeedForwardSpec, GatedUnitSpec, HeadSpec, LayerSpec, ModelSpec,
                          NoFeedForwardSpec, NormSpec, PositionSpec, RetentionSpec, RotarySpec, RunEntry,
                          ScoreRoutedExpertsSpec)
from ..registry import Architecture, register_architecture


def _norm(c, name):
    return NormSpec("rmsnorm", c.width, c.norm_eps, name)


def _unit(prefix, ff, activation):
    return GatedUnitSpec(ff, 0.0, prefix + "gate", prefix + "up", prefix + "down", alpha=1.0, activation=activation)


def _rotary(m):
    if m.rot is None:
        return None
    return RotarySpec("rotary", head_dim=m.dim, dims=m.rot.dims, base=m.rot.base, interleaved=False)


def _kept_keys(c: ZokanexConfig, i: int):
    """What layer i's cache must keep: the widest window among its own mask and the masks of the layers that read it."""
    masks = [c.layers[i].mixer.mask_size] + [l.mixer.mask_size for l in c.layers
                                             if l.type == "attention" and l.mixer.kv_from == i]
    return "all" if any(m is None for m in masks) else max(masks)


def _mixer_spec(c: ZokanexConfig, i: int):
    layer, p = c.layers[i], f"l{i}."
    m = layer.mixer
    if layer.type == "retention":
        return RetentionSpec("retention", width=c.width, n_heads=m.heads, head_dim=m.dim, value_dim=m.vdim, decay=m.decay,
                             key_scale=m.dim ** -0.5, norm_eps=c.norm_eps, query_weight=p + "mix.q", key_weight=p + "mix.k",
                             value_weight=p + "mix.v", gate_weight=p + "mix.g", out_weight=p + "mix.o", rotary=_rotary(m))
    own = m.kv_from is None
    return AttentionSpec("attention", width=c.width, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, scale=m.scale,
                         window=m.mask_size, qkv_weight=(p + "mix.q", p + "mix.k", p + "mix.v") if own else (p + "mix.q",),
                         qkv_bias=None, out_weight=p + "mix.o", out_bias=None, value_dim=m.vdim, rotary=_rotary(m),
                         query_norm=p + "mix.q.norm", key_norm=p + "mix.k.norm" if own else None, head_norm_eps=c.norm_eps,
                         own_keys_values=own, keep_window=_kept_keys(c, i) if own else None)


def _feed_forward_spec(c: ZokanexConfig, i: int):
    f, p = c.layers[i].mlp, f"l{i}.mlp."
    if f is None:
        return NoFeedForwardSpec()
    if f.kind == "dense":
        return GatedFeedForwardSpec("gated", c.width, _unit(p, f.ff, "gelu_tanh"))
    return ScoreRoutedExpertsSpec(
        "experts_by_score", width=c.width, top=f.top, router=p + "router",
        experts=tuple(_unit(f"{p}e{e}.", f.ff, "silu") for e in range(f.experts)), groups=f.groups, keep_groups=f.keep,
        weight_scale=f.scale, score="sigmoid", shared=None if f.shared_ff is None else _unit(p + "shared.", f.shared_ff, "silu"),
        shared_gate=None if f.shared_ff is None else p + "shared.sg")


def build_spec(c: ZokanexConfig) -> ModelSpec:
    layers = tuple(LayerSpec("parallel", _mixer_spec(c, i), _feed_forward_spec(c, i), (_norm(c, f"l{i}.norm1"),))
                   for i in range(len(c.layers)))
    # every layer is one stop of the run order; a layer without keys and values reads the stop of the layer it names
    run_order = tuple(RunEntry(i, getattr(layer.mixer, "kv_from", None)) for i, layer in enumerate(c.layers))
    return ModelSpec(
        architecture=ARCHITECTURE, vocab_size=c.vocab, width=c.width, max_positions=None,
        embedding=EmbeddingSpec("tokens", c.vocab, c.width, table="embed", scale=c.embedding_scale),
        position=PositionSpec("none", 0, c.width), layers=layers, run_order=run_order,
        head=HeadSpec("linear", c.vocab, c.width, norm=_norm(c, "final.norm"), weight="head"),
        eos_token_ids=tuple(c.eos_token_ids))


def random_tensors(c: ZokanexConfig, seed: int, matrix_dtype=torch.float32, device="cpu") -> dict:
    """Seeded random weights under their checkpoint names, in a fixed draw order: the token table ~N(0, 1/width)
    (so that table x sqrt(width) has unit entries), matrices ~N(0, 1/in), norm weights ~N(1, 0.1)."""
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    out = {}

    def matrix(name, rows, cols, gain=1.0):
        out[name] = (torch.randn((rows, cols), generator=g, dtype=torch.float32, device=device) * gain / math.sqrt(cols)).to(matrix_dtype)

    def vector(name, n):
        out[name] = 1.0 + torch.randn((n,), generator=g, dtype=torch.float32, device=device) * 0.1

    def unit(prefix, ff):
        matrix(prefix + "gate", ff, c.width)
        matrix(prefix + "up", ff, c.width)
        matrix(prefix + "down", c.width, ff)

    matrix("embed", c.vocab, c.width)
    for i, layer in enumerate(c.layers):
        p, m = f"l{i}.", layer.mixer
        vector(p + "norm1", c.width)
        matrix(p + "mix.q", m.heads * m.dim, c.width)
        if layer.type == "attention":
            vector(p + "mix.q.norm", m.dim)
            if m.kv_from is None:
                matrix(p + "mix.k", m.kv_heads * m.dim, c.width)
                matrix(p + "mix.v", m.kv_heads * m.vdim, c.width)
                vector(p + "mix.k.norm", m.dim)
        else:
            matrix(p + "mix.k", m.heads * m.dim, c.width)
            matrix(p + "mix.v", m.heads * m.vdim, c.width)
            matrix(p + "mix.g", m.heads * m.vdim, c.width)
        matrix(p + "mix.o", c.width, m.heads * m.vdim)
        f = layer.mlp
        if f is None:
            continue
        if f.kind == "dense":
            unit(p + "mlp.", f.ff)
            continue
        for e in range(f.experts):
            unit(f"{p}mlp.e{e}.", f.ff)
        matrix(p + "mlp.router", f.experts, c.width, gain=2.0)
        if f.shared_ff is not None:
            unit(p + "mlp.shared.", f.shared_ff)
            matrix(p + "mlp.shared.sg", 1, c.width)
    vector("final.norm", c.width)
    matrix("head", c.vocab, c.width)
    return out


register_architecture(Architecture(ARCHITECTURE, ZokanexConfig.from_dict, build_spec, random_tensors), replace=True)
