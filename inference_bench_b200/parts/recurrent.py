"""A gated linear recurrence as a mixer (the HGRN2 form): linear attention in which the forget gate also decides what is written.

With h the layer's input, per token and head (q, f of size `dim`, v of size `vdim`):
    q = silu(Wq h),   f = lower + (1 - lower) * sigmoid(Wf h + b_f),   v = Wv h
    S <- diag(f) S + (1 - f) v^T        (S [dim, vdim]: the request's state, float32, zero at admission)
    o = S^T q;   every head's o is divided by its root mean square over vdim and scaled by one weight vector shared by the heads;
    out = Wo [o_1 | o_2 | ...]
There is no key and no scale. The three projections are one matrix product [q | f | v]; gates, state, o and the norm are float32
whatever the activation dtype. The state is a fixed-size slot per request (`FixedState`), read and written by the kernel through the
device copy of the step's slots, so a step of decoded tokens can be captured.

A segment of more than `ops.RECURRENCE_CHUNK` tokens (a prompt portion) is cut into chunks that are walked side by side, each from a zero
state; their states are then carried from chunk to chunk and every chunk's incoming state is applied to its rows: the same sums in
another order, with as many CTAs as chunks. Shorter segments (decoded tokens among them) are walked token by token. Which way a segment
goes depends on its own length only, so a request's result does not depend on what shares its step.
"""
from __future__ import annotations

import torch

import numpy as np

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
        short, long_segs, chunks = self._cut(ctx)
        ops.gated_recurrence(proj, self.f_bias, self.lower, cache.tensor, ctx.seg_start, ctx.seg_slot, ctx.n_segments, o, self.heads, self.dim, self.vdim,
                             seg_list=short, long_segs=long_segs, chunks=chunks)
        normed = rt.empty((T, self.heads * self.vdim))
        ops.head_rmsnorm(o, self.o_norm, self.norm_eps, normed)
        return rt.linear(normed, self.wo)

    @staticmethod
    def _cut(ctx):
        """(segments walked token by token or None for all, long segments [n, 3], their chunks [m, 2]) on the device; one table a step for all layers."""
        if ctx.fixed_shape:
            return None, None, None
        if "recurrence cut" not in ctx.memo:
            C = ops.RECURRENCE_CHUNK
            starts = ctx.h_seg_start
            lens = np.diff(starts)
            if not (lens > C).any():
                ctx.memo["recurrence cut"] = (None, None, None)
            else:
                short = np.nonzero(lens <= C)[0].astype(np.int32)
                long_segs, chunks = [], []
                for s in np.nonzero(lens > C)[0].tolist():
                    first = len(chunks)
                    chunks += [(t, min(C, int(starts[s + 1]) - t)) for t in range(int(starts[s]), int(starts[s + 1]), C)]
                    long_segs.append((s, first, len(chunks) - first))
                flat = np.concatenate([short, np.asarray(long_segs, np.int32).ravel(), np.asarray(chunks, np.int32).ravel()]).astype(np.int32)
                dev = torch.from_numpy(flat).pin_memory().to(ctx.rt.device, non_blocking=True)
                a, b = short.size, short.size + 3 * len(long_segs)
                ctx.memo["recurrence cut"] = (dev[:a], dev[a:b].view(-1, 3), dev[b:].view(-1, 2))
        return ctx.memo["recurrence cut"]
