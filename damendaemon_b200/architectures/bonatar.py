"""Bonatar described with the framework's parts.

A decoder of pre-norm layers over a float32 stream that starts as the token's row times a scale. Norms are RMS
norms whose weight is stored around zero (factor 1 + w). A layer's mixer is grouped-query attention with separate
query/key and value head sizes, rotary positions on the first dimensions of every query and key head (neighbouring
dimensions paired; frequencies blended for a long context), a mask of chunks counted from the start of the sequence
and a sigmoid gate per head on the attention's output. Its feed-forward is dense (the square of relu between two
matrices), or a set of small gated units of which a table of token ids chooses each token's, with a shared unit beside
them, or absent. A layer may run the tensors of an earlier one, with a cache of its own: the run order names that
layer again. The final norm and an untied head give the logits.

Tensor names: embed, l<i>.norm1, l<i>.norm2, l<i>.mix.{q,k,v,g,o}, l<i>.mlp.{up,down} or
l<i>.mlp.{table, e<j>.{gate,up,down}, shared.{gate,up,down}}, final.norm, head; matrices [out, in].
"""
from __future__ import annotations

import math

import torch

from ..config.bonatar import ARCHITECTURE, BonatarConfig
from ..parts.spec import (AttentionSpec, DenseFeedForwardSpec, EmbeddingSpec, GatedUnitSpec, HeadSpec, LayerSpec,
                          LongContextBlend, ModelSpec, NoFeedForwardSpec, NormSpec, PositionSpec, RotarySpec, RunEntry,
                          TableRoutedExpertsSpec)
from ..registry import Architecture, register_architecture

GATE_SLOPE = 1.702      # the gated unit's sigmoid is taken of this many times the clamped gate


def _norm(c, name):
    return NormSpec("rmsnorm", c.width, c.norm_eps, name, weight_offset=1.0)


def _unit(prefix, unit):
    return GatedUnitSpec(unit.ff, unit.limit, prefix + "gate", prefix + "up", prefix + "down", alpha=GATE_SLOPE)


def _layer_spec(c: BonatarConfig, i: int) -> LayerSpec:
    layer, p = c.layers[i], f"l{i}."
    m = layer.mixer
    rotary = None
    if m.rot is not None:
        s = m.rot.scaling
        rotary = RotarySpec("rotary", head_dim=m.dim, dims=m.rot.dims, base=m.rot.base, interleaved=True,
                            blend=None if s is None else LongContextBlend(s.factor, s.original, s.fast, s.slow))
    mixer = AttentionSpec("attention", width=c.width, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim,
                          scale=m.scale, window=None, qkv_weight=(p + "mix.q", p + "mix.k", p + "mix.v"), qkv_bias=None,
                          out_weight=p + "mix.o", out_bias=None, value_dim=m.vdim, chunk=m.mask_size,
                          gate_weight=p + "mix.g", rotary=rotary)
    if layer.mlp is None:
        return LayerSpec("pre_norm_mixer", mixer, NoFeedForwardSpec(), (_norm(c, p + "norm1"),))
    if layer.mlp.kind == "dense":
        feed = DenseFeedForwardSpec("dense", width=c.width, inner=layer.mlp.ff, activation="relu2", up_weight=p + "mlp.up",
                                    up_bias=None, down_weight=p + "mlp.down", down_bias=None)
    else:
        feed = TableRoutedExpertsSpec(
            "experts_by_table", width=c.width, vocab_size=c.vocab, top=layer.mlp.top, table=p + "mlp.table",
            experts=tuple(_unit(f"{p}mlp.e{e}.", layer.mlp.expert) for e in range(layer.mlp.experts)),
            shared=None if layer.mlp.shared is None else _unit(p + "mlp.shared.", layer.mlp.shared))
    return LayerSpec("pre_norm", mixer, feed, (_norm(c, p + "norm1"), _norm(c, p + "norm2")))


def build_spec(c: BonatarConfig) -> ModelSpec:
    # layers with tensors of their own become the model's layers; the run order names a layer again where another
    # entry runs its tensors (every stop of the run order has a cache of its own)
    own = [i for i, layer in enumerate(c.layers) if layer.weights_of is None]
    index = {i: n for n, i in enumerate(own)}
    run_order = tuple(RunEntry(index[i if layer.weights_of is None else layer.weights_of]) for i, layer in enumerate(c.layers))
    return ModelSpec(
        architecture=ARCHITECTURE, vocab_size=c.vocab, width=c.width, max_positions=None,
        embedding=EmbeddingSpec("tokens", c.vocab, c.width, table="embed", scale=c.embedding_scale),
        position=PositionSpec("none", 0, c.width),
        layers=tuple(_layer_spec(c, i) for i in own), run_order=run_order,
        head=HeadSpec("linear", c.vocab, c.width, norm=_norm(c, "final.norm"), weight="head"),
        eos_token_ids=tuple(c.eos_token_ids))


def random_tensors(c: BonatarConfig, seed: int, matrix_dtype=torch.float32, device="cpu") -> dict:
    """Seeded random weights under their checkpoint names, in a fixed draw order: the token table ~N(0, 1/width)
    (so that table x sqrt(width) has unit entries), matrices ~N(0, 1/in), norm weights ~N(0, 0.1) around zero,
    tables of distinct experts per token id."""
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    out = {}

    def matrix(name, rows, cols, gain=1.0):
        out[name] = (torch.randn((rows, cols), generator=g, dtype=torch.float32, device=device) * gain / math.sqrt(cols)).to(matrix_dtype)

    def vector(name, n):
        out[name] = torch.randn((n,), generator=g, dtype=torch.float32, device=device) * 0.1

    def unit(prefix, u):
        matrix(prefix + "gate", u.ff, c.width)
        matrix(prefix + "up", u.ff, c.width)
        matrix(prefix + "down", c.width, u.ff)

    matrix("embed", c.vocab, c.width)
    for i, layer in enumerate(c.layers):
        if layer.weights_of is not None:
            continue
        p, m = f"l{i}.", layer.mixer
        vector(p + "norm1", c.width)
        matrix(p + "mix.q", m.heads * m.dim, c.width)
        matrix(p + "mix.k", m.kv_heads * m.dim, c.width)
        matrix(p + "mix.v", m.kv_heads * m.vdim, c.width)
        matrix(p + "mix.g", m.heads, c.width)
        matrix(p + "mix.o", c.width, m.heads * m.vdim)
        if layer.mlp is None:
            continue
        vector(p + "norm2", c.width)
        if layer.mlp.kind == "dense":
            matrix(p + "mlp.up", layer.mlp.ff, c.width)
            matrix(p + "mlp.down", c.width, layer.mlp.ff)
        else:
            for e in range(layer.mlp.experts):
                unit(f"{p}mlp.e{e}.", layer.mlp.expert)
            scores = torch.rand((c.vocab, layer.mlp.experts), generator=g, device=device)
            out[p + "mlp.table"] = scores.argsort(dim=1)[:, :layer.mlp.top].to(torch.int32).contiguous()
            if layer.mlp.shared is not None:
                unit(p + "mlp.shared.", layer.mlp.shared)
    vector("final.norm", c.width)
    matrix("head", c.vocab, c.width)
    return out


register_architecture(Architecture(ARCHITECTURE, BonatarConfig.from_dict, build_spec, random_tensors), replace=True)
