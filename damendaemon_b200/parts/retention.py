"""The retention mixer: linear attention with a fixed decay per head and no softmax, over per-request state.

One fused projection gives queries, keys, values and the output gate. Per head, S <- decay * S + k' v^T and
o = S^T q' token by token, with q', k' rotated (the spec's rotary encoding) and k' scaled; the state S is float32 and
lives in the request's state slot (a ``RequestState`` need, zeroed when the slot is taken), so a portion of a prompt
continues exactly where the portion before stopped and a decoded token where the prompt stopped. Every head's o is
divided by its root mean square, multiplied by silu(gate) and projected, the residual add in the last product's
epilogue. Everything between the projection's output and the operand of the output projection is float32.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.manager import RequestState
from .interfaces import Mixer
from .linear import linear
from .registry import POSITIONS, lookup, register_mixer
from .spec import TensorDecl


def _names(spec):
    return (spec.query_weight, spec.key_weight, spec.value_weight, spec.gate_weight)


@register_mixer("retention")
class Retention(Mixer):
    graph_safe = True

    def __init__(self, spec, weights, runtime):
        self.spec, self.runtime = spec, runtime
        if len(spec.decay) != spec.n_heads:
            raise ValueError(f"{len(spec.decay)} decays for {spec.n_heads} heads")
        if spec.head_dim > 256:
            raise ValueError(f"a retention head of {spec.head_dim} is not supported (at most 256)")
        key = "+".join(_names(spec))
        self.proj_w = weights[key]
        if self.proj_w.shape[0] % 8:
            # rows of zeros make the projection's row stride a multiple of eight elements (their outputs are never read)
            pad = torch.zeros((-self.proj_w.shape[0] % 8, self.proj_w.shape[1]), dtype=self.proj_w.dtype, device=self.proj_w.device)
            self.proj_w = weights[key] = torch.cat([self.proj_w, pad], dim=0)
        self.out_w = weights[spec.out_weight]
        self.qk_width, self.v_width = spec.n_heads * spec.head_dim, spec.n_heads * spec.value_dim
        self.decay = torch.tensor(spec.decay, dtype=torch.float32, device=runtime.device)
        self.rotary = None if spec.rotary is None else lookup(POSITIONS, spec.rotary, "position encoding")(spec.rotary, weights, runtime)
        if self.rotary is not None and self.rotary.magnitude != 1.0:
            raise ValueError("retention takes plain rotary frequencies (no scaled cosines)")

    @staticmethod
    def tensor_decls(spec):
        qk, v = spec.n_heads * spec.head_dim, spec.n_heads * spec.value_dim
        shapes = ((qk, spec.width), (qk, spec.width), (v, spec.width), (v, spec.width))
        return [TensorDecl("+".join(_names(spec)), (2 * qk + 2 * v, spec.width), "matrix", False, tuple(zip(_names(spec), shapes))),
                TensorDecl(spec.out_weight, (spec.width, v), "matrix")]

    @staticmethod
    def cache_needs(spec):
        # the state lies as the kernel's warps hold it, so that they read and write whole lines
        return [RequestState(kernels.retention_state_shape(spec.n_heads, spec.head_dim, spec.value_dim), "float32")]

    def forward(self, y, residual, ctx, cache, position):
        s, a, b = self.spec, self.qk_width, self.v_width
        if cache.state is None:
            raise ValueError("the retention mixer needs its per-request state (a stop of the run order with a cache of its own)")
        proj = linear(self.runtime, y, self.proj_w)
        q, k, v, gate = proj[:, :a], proj[:, a:2 * a], proj[:, 2 * a:2 * a + b], proj[:, 2 * a + b:2 * a + 2 * b]
        o = kernels.retention(q, k, v, ctx.positions, ctx.entry_start, ctx.entry_slot, self.decay, s.key_scale, cache.state,
                              s.head_dim, s.value_dim, freqs=None if self.rotary is None else self.rotary.freqs,
                              interleaved=True if self.rotary is None else self.rotary.spec.interleaved)
        mixed = kernels.retention_finish(o, gate, s.n_heads, s.norm_eps, proj.dtype)
        return linear(self.runtime, mixed, self.out_w, residual=residual, out_dtype=residual.dtype, out=residual)
