"""Feed-forwards. Dense two-matrix MLP with the activation fused into the first product's
epilogue and the residual add into the second's (damendaemon/gpt2.py:62-64). Experts chosen by a
table of token ids: small gated units, a token's chosen ones weighted equally, a shared one for every
token; their products run grouped, expert by expert, over rows sorted on the device. Experts chosen
by a router's scores: the same grouped products after a routing kernel, each chosen expert weighted by its
score. 'gated': one dense gated unit. 'none': a layer without a feed-forward."""
from __future__ import annotations

import torch

from .. import kernels
from .interfaces import FeedForward
from .linear import grouped_gated_unit, grouped_linear, grouped_on_tensor_cores, grouped_tile, linear
from .registry import register_feed_forward
from .spec import TensorDecl

ACTIVATIONS = ("gelu_new", "gelu", "relu2")


@register_feed_forward("dense")
class DenseFeedForward(FeedForward):
    graph_safe = True

    def __init__(self, spec, weights, runtime):
        if spec.activation not in ACTIVATIONS:
            raise ValueError(f"activation {spec.activation!r} is not supported; known: {ACTIVATIONS}")
        self.spec, self.runtime = spec, runtime
        self.up_w, self.down_w = weights[spec.up_weight], weights[spec.down_weight]
        self.up_b = weights[spec.up_bias] if spec.up_bias else None
        self.down_b = weights[spec.down_bias] if spec.down_bias else None

    @staticmethod
    def tensor_decls(spec):
        io = spec.stored_in_out
        decls = [TensorDecl(spec.up_weight, (spec.width, spec.inner) if io else (spec.inner, spec.width), "matrix", io),
                 TensorDecl(spec.down_weight, (spec.inner, spec.width) if io else (spec.width, spec.inner), "matrix", io)]
        if spec.up_bias:
            decls.append(TensorDecl(spec.up_bias, (spec.inner,), "vector"))
        if spec.down_bias:
            decls.append(TensorDecl(spec.down_bias, (spec.width,), "vector"))
        return decls

    def forward(self, y, residual, ctx):
        hidden = linear(self.runtime, y, self.up_w, self.up_b, activation=self.spec.activation)
        return linear(self.runtime, hidden, self.down_w, self.down_b, residual=residual, out_dtype=residual.dtype,
                      out=residual)


@register_feed_forward("none")
class NoFeedForward(FeedForward):
    graph_safe = True

    def __init__(self, spec, weights, runtime):
        self.spec = spec

    def forward(self, y, residual, ctx):
        return residual


def _unit_decls(unit, width):
    return [TensorDecl(unit.gate_weight, (unit.inner, width), "matrix"),
            TensorDecl(unit.up_weight, (unit.inner, width), "matrix"),
            TensorDecl(unit.down_weight, (width, unit.inner), "matrix")]


@register_feed_forward("experts_by_table")
class TableRoutedExperts(FeedForward):
    """out = residual + (1/K) sum over the K experts of row ids[t] of the table of unit_e(y) + shared(y).

    The experts' gate and up matrices are stacked [E, 2 * inner, width] (gate rows, then up rows) and their down
    matrices [E, width, inner] once, when the part is built. A step sorts its (token, choice) pairs by expert on the
    device (kernels.route_by_table: every expert's rows start on a multiple of the product's row tile), gathers the
    normed rows in that order, runs two grouped products (on the tensor cores the first computes gate and up together
    and applies the gated unit in its epilogue; else the unit is a kernel between them) and adds each token's rows, in
    the order of its choices, into the float32 stream. Launch shapes depend on the step's counts only, so a step
    can be replayed from a graph."""
    graph_safe = True

    def __init__(self, spec, weights, runtime):
        self.spec, self.runtime = spec, runtime
        first = spec.experts[0]
        if any((u.inner, u.limit, u.alpha) != (first.inner, first.limit, first.alpha) for u in spec.experts):
            raise ValueError("the experts of one layer must have one size, limit and slope")
        if not 0 < spec.top <= len(spec.experts):
            raise ValueError(f"{spec.top} experts per token of {len(spec.experts)}")
        self.table = weights[spec.table]
        self.tensor_cores = grouped_on_tensor_cores(runtime, runtime.dtype, spec.width, first.inner)
        self.gate_up = torch.stack([torch.cat([weights[u.gate_weight], weights[u.up_weight]], dim=0) for u in spec.experts])
        self.down = torch.stack([weights[u.down_weight] for u in spec.experts])
        # the stacks take the place of the single matrices (one copy on the device, and in the engine's count of bytes)
        for u in spec.experts:
            for name in (u.gate_weight, u.up_weight, u.down_weight):
                weights.pop(name, None)
        weights[spec.table + ":gate_up"], weights[spec.table + ":down"] = self.gate_up, self.down
        self.shared = None
        if spec.shared is not None:
            u = spec.shared
            joined = torch.cat([weights.pop(u.gate_weight), weights.pop(u.up_weight)], dim=0).contiguous()
            weights[spec.table + ":shared_gate_up"] = joined
            self.shared = (joined, weights[u.down_weight])

    @staticmethod
    def tensor_decls(spec):
        decls = [TensorDecl(spec.table, (spec.vocab_size, spec.top), "int")]
        for unit in spec.experts:
            decls += _unit_decls(unit, spec.width)
        if spec.shared is not None:
            decls += _unit_decls(spec.shared, spec.width)
        return decls

    def forward(self, y, residual, ctx):
        s, rt = self.spec, self.runtime
        unit = s.experts[0]
        if self.shared is not None:
            gate_up = linear(rt, y, self.shared[0])
            hidden = kernels.gated_unit(gate_up, s.shared.limit, s.shared.alpha, form=s.shared.activation)
            residual = linear(rt, hidden, self.shared[1], residual=residual, out_dtype=residual.dtype, out=residual)
        tile = grouped_tile(self.tensor_cores, y.shape[0] * s.top, len(s.experts))
        pair_row, row_token, tile_group = kernels.route_by_table(ctx.token_ids, self.table, len(s.experts), tile)
        rows = kernels.gather_rows(y, row_token)
        hidden = grouped_gated_unit(self.tensor_cores, rows, self.gate_up, tile_group, tile, unit.limit, unit.alpha, unit.activation)
        out = grouped_linear(self.tensor_cores, hidden, self.down, tile_group, tile, out_dtype=torch.float32)
        return kernels.combine_rows(out, pair_row, residual, s.top, 1.0 / s.top)


def _check_unit(unit):
    if unit.activation not in kernels.GATED_FORMS:
        raise ValueError(f"gated unit activation {unit.activation!r} is not supported; known: {sorted(kernels.GATED_FORMS)}")


@register_feed_forward("gated")
class GatedFeedForward(FeedForward):
    """residual + W_down f(W_gate y, W_up y): gate and up are one product (their matrices joined at load), the unit's
    value is computed in float32 from its two halves, the residual add is the last product's epilogue."""
    graph_safe = True

    def __init__(self, spec, weights, runtime):
        self.spec, self.runtime = spec, runtime
        _check_unit(spec.unit)
        self.gate_up = weights[spec.unit.gate_weight + "+" + spec.unit.up_weight]
        self.down = weights[spec.unit.down_weight]

    @staticmethod
    def tensor_decls(spec):
        u = spec.unit
        piece = (u.inner, spec.width)
        return [TensorDecl(u.gate_weight + "+" + u.up_weight, (2 * u.inner, spec.width), "matrix", False,
                           ((u.gate_weight, piece), (u.up_weight, piece))),
                TensorDecl(u.down_weight, (spec.width, u.inner), "matrix")]

    def forward(self, y, residual, ctx):
        u = self.spec.unit
        hidden = kernels.gated_unit(linear(self.runtime, y, self.gate_up), u.limit, u.alpha, form=u.activation)
        return linear(self.runtime, hidden, self.down, residual=residual, out_dtype=residual.dtype, out=residual)


@register_feed_forward("experts_by_score")
class ScoreRoutedExperts(FeedForward):
    """out = residual + sum over a token's chosen experts of weight_e * unit_e(y) + gate * shared(y).

    One kernel (kernels.route_by_score, a warp a token) computes the router's logits as float32 sums (its matrix and, as
    one more row, the shared unit's gate vector) and turns them into the token's experts, their weights and the shared
    unit's gate.
    From there on the step is that of experts chosen by a table: the (token, choice) pairs sorted by expert on the
    device, the normed rows gathered in that order, two grouped products (on the tensor cores the first with the gated
    unit in its epilogue), and each token's rows added, weighted, in the order of its choices, into the float32 stream.
    The shared unit's gate multiplies its hidden row before the down product, whose epilogue adds into the stream.
    Launch shapes depend on the step's counts only, so a step can be replayed from a graph."""
    graph_safe = True

    def __init__(self, spec, weights, runtime):
        self.spec, self.runtime = spec, runtime
        first = spec.experts[0]
        for u in spec.experts + ((spec.shared,) if spec.shared else ()):
            _check_unit(u)
        if any((u.inner, u.limit, u.alpha, u.activation) != (first.inner, first.limit, first.alpha, first.activation) for u in spec.experts):
            raise ValueError("the experts of one layer must have one size and one form")
        E = len(spec.experts)
        if not 0 < spec.top <= E or spec.groups <= 0 or E % spec.groups or not 0 < spec.keep_groups <= spec.groups or \
                spec.top > E // spec.groups * spec.keep_groups:
            raise ValueError(f"{spec.top} experts per token of {E} in {spec.groups} groups of which {spec.keep_groups} stay")
        if spec.score != "sigmoid":
            raise ValueError(f"router score {spec.score!r} is not supported; known: ['sigmoid']")
        if spec.shared_gate and spec.shared is None:
            raise ValueError("a shared unit's gate without a shared unit")
        self.router = weights[self._router_key(spec)]
        self.tensor_cores = grouped_on_tensor_cores(runtime, runtime.dtype, spec.width, first.inner)
        self.gate_up = torch.stack([torch.cat([weights[u.gate_weight], weights[u.up_weight]], dim=0) for u in spec.experts])
        self.down = torch.stack([weights[u.down_weight] for u in spec.experts])
        # the stacks take the place of the single matrices (one copy on the device, and in the engine's count of bytes)
        for u in spec.experts:
            for name in (u.gate_weight, u.up_weight, u.down_weight):
                weights.pop(name, None)
        weights[spec.router + ":gate_up"], weights[spec.router + ":down"] = self.gate_up, self.down
        self.shared = None
        if spec.shared is not None:
            u = spec.shared
            joined = torch.cat([weights.pop(u.gate_weight), weights.pop(u.up_weight)], dim=0).contiguous()
            weights[spec.router + ":shared_gate_up"] = joined
            self.shared = (joined, weights[u.down_weight])

    @staticmethod
    def _router_key(spec):
        return spec.router + "+" + spec.shared_gate if spec.shared_gate else spec.router

    @staticmethod
    def tensor_decls(spec):
        E = len(spec.experts)
        if spec.shared_gate:
            decls = [TensorDecl(spec.router + "+" + spec.shared_gate, (E + 1, spec.width), "matrix", False,
                                ((spec.router, (E, spec.width)), (spec.shared_gate, (1, spec.width))))]
        else:
            decls = [TensorDecl(spec.router, (E, spec.width), "matrix")]
        for unit in spec.experts:
            decls += _unit_decls(unit, spec.width)
        if spec.shared is not None:
            decls += _unit_decls(spec.shared, spec.width)
        return decls

    def forward(self, y, residual, ctx):
        s, rt = self.spec, self.runtime
        unit, E = s.experts[0], len(s.experts)
        # the router's logits (float32 sums of exact products, whatever the storage type) and the choice, in one kernel
        chosen, pair_weight, shared_gate = kernels.route_by_score(y, self.router, E, s.top, s.groups, s.keep_groups, s.weight_scale,
                                                                  shared_gate=bool(s.shared_gate))
        if self.shared is not None:
            hidden = kernels.gated_unit(linear(rt, y, self.shared[0]), s.shared.limit, s.shared.alpha, form=s.shared.activation,
                                        row_scale=shared_gate)
            residual = linear(rt, hidden, self.shared[1], residual=residual, out_dtype=residual.dtype, out=residual)
        tile = grouped_tile(self.tensor_cores, y.shape[0] * s.top, E)
        pair_row, row_token, tile_group = kernels.route_by_table(None, chosen, E, tile)
        rows = kernels.gather_rows(y, row_token)
        hidden = grouped_gated_unit(self.tensor_cores, rows, self.gate_up, tile_group, tile, unit.limit, unit.alpha, unit.activation)
        out = grouped_linear(self.tensor_cores, hidden, self.down, tile_group, tile, out_dtype=torch.float32)
        return kernels.combine_rows(out, pair_row, residual, s.top, 1.0, pair_weight=pair_weight.view(-1))
