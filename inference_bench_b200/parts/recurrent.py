"""A gated linear recurrence as a mixer (the HGRN2 form): linear attention in which the forget gate also decides what is written.

With h the layer's input, per token and head (q, f of size `dim`, v of size `vdim`):
    q = silu(Wq h),   f = lower + (1 - lower) * sigmoid(Wf h + b_f),   v = Wv h
    S <- diag(f) S + (1 - f) v^T        (S [dim, vdim]: the request's state, float32, zero at admission)
    o = S^T q;   every head's o is divided by its root mean square over vdim and scaled by one weight vector shared by the heads;
    out = Wo [o_1 | o_2 | ...]
There is no key and no scale. The three projections are one matrix product [q | f | v]; gates, state, o and the norm are float32
whatever the activation dtype. The state is a fixed-size slot per request (`FixedState`), read and written by the kernel through the
device copy of the step's slots, so a step of decoded tokens can be captured.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from . import base
from .base import FixedState, WeightSpec


@base.register_mixer("hgrn2")
class GatedLinearRecurrence(base.Mixer):
    def __init__(self, prefix: str, hidden: int, heads: int, dim: int, vdim: int, norm_eps: float,
                 names: tuple = ("q", "f", "f.b", "lower", "v", "norm", "o")):
        if heads <= 0 or dim <= 0 or vdim <= 0:
            raise ValueError(f"heads {heads}, dim {dim} and vdim {vdim} must be positive")
        if dim > 512:
            raise ValueError(f"a head's key size {dim} is above the 512 the recurrence kernel holds")
        self.prefix, self.hidden, self.heads, self.dim, self.vdim, self.norm_eps, self.names = prefix, hidden, heads, dim, vdim, norm_eps, tuple(names)
        self.w_in = self.wo = self.f_bias = self.lower = self.o_norm = None

    def cache_need(self):
        return FixedState((self.heads, self.dim, self.vdim), torch.float32)

    def _n(self, i: int) -> str:
        return f"{self.prefix}.{self.names[i]}"

    def weight_specs(self):
        H, D, V = self.heads, self.dim, self.vdim
        return [WeightSpec(self._n(0), (H * D, self.hidden)), WeightSpec(self._n(1), (H * D, self.hidden)), WeightSpec(self._n(2), (H * D,), std=0.5),
                WeightSpec(self._n(3), (H * D,), role="gate_floor"), WeightSpec(self._n(4), (H * V, self.hidden)), WeightSpec(self._n(5), (V,), role="norm"),
                WeightSpec(self._n(6), (self.hidden, H * V))]

    def bind(self, weights, rt):
        self.w_in = rt.matrix(torch.cat([weights[self._n(0)], weights[self._n(1)], weights[self._n(4)]], dim=0))   # [q | f | v] rows: one product
        self.f_bias, self.lower, self.o_norm = rt.vector(weights[self._n(2)]), rt.vector(weights[self._n(3)]), rt.vector(weights[self._n(5)])
        self.wo = rt.matrix(weights[self._n(6)])

    def forward(self, ctx, h, cache):
        rt, T = ctx.rt, ctx.n_tokens
        proj = rt.linear(h, self.w_in)
        o = rt.empty((T, self.heads, self.vdim), torch.float32)
        ops.gated_recurrence(proj, self.f_bias, self.lower, cache.tensor, ctx.seg_start, ctx.seg_slot, ctx.n_segments, o, self.heads, self.dim, self.vdim)
        normed = rt.empty((T, self.heads * self.vdim))
        ops.head_rmsnorm(o, self.o_norm, self.norm_eps, normed)
        return rt.linear(normed, self.wo)
