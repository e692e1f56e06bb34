"""A pre-norm block whose sublayers read their input through a short causal convolution over time, whose contributions are scaled
per channel, and whose result is mixed with the results of all earlier layers.

Layer i (counted from 0), with x the stream it is given, X_0 the embedding's output and X_(j+1) the result of layer j:
    h = norm1(x);  h <- h + conv1(h);  x <- x + ls1 * (mixer(h) + the mixer's output bias)
    h = norm2(x);  h <- h + conv2(h);  x <- x + ls2 * feed_forward(h)            (a layer may have no feed-forward)
    X_(i+1) = x;   x <- sum_{j <= i+1} dwa[j] * X_j                               (the depth-weighted average goes on to layer i + 1)
conv(h)_t = sum_k w[:, k] * h_(t - taps + 1 + k) per channel, zeros before a request's first token. The last taps - 1 normed rows of
a request, for each of the two sublayers, are state (a fixed-size slot per request, beside the mixer's own cache or state).

Kernels (csrc/layernorm.cu; a step whose requests all bring one token runs the first two as one, `add_layernorm_conv_single`): `add_layernorm` adds the contribution before it with its scale and bias, norms, and lays the normed rows
out with every request's state rows in front of its tokens; `causal_conv_rows` convolves, rounds to the activation dtype and writes
the new state; `depth_average` adds the feed-forward's contribution, files X_(i+1) and mixes. The results X_j of a step live in one
buffer [layers + 1, T, H] kept in the step's memo.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from . import base
from .base import FixedState, Several, WeightSpec
from .standard import NoFeedForward


@base.register_block("prenorm_canon")
class CanonBlock(base.Block, base.Part):
    takes_out_bias = True

    def __init__(self, mixer_norm, mixer, feed_forward_norm, feed_forward, prefix: str, hidden: int, taps: int, index: int, depth: int,
                 names: tuple = ("ls1", "ls2", "canon1", "canon2", "dwa")):
        """index: this layer's number; depth: the number of layers (the buffer of results has depth + 1 entries); taps: the convolution's
        length (1: no convolution state)."""
        base.Block.__init__(self, mixer_norm, mixer, feed_forward_norm, feed_forward)
        if taps < 1 or not 0 <= index < depth:
            raise ValueError(f"taps {taps} must be at least 1 and layer {index} one of {depth}")
        self.has_ff = not isinstance(feed_forward, NoFeedForward)
        for norm in (mixer_norm, feed_forward_norm) if self.has_ff else (mixer_norm,):
            if not getattr(norm, "takes_layout", False):
                raise ValueError(f"this arrangement needs norms that lay their rows out for the convolution (layernorm does); {type(norm).__name__} does not")
        self.prefix, self.hidden, self.taps, self.index, self.depth, self.names = prefix, hidden, taps, index, depth, tuple(names)
        self.ls1 = self.ls2 = self.conv1 = self.conv2 = self.mix = None

    # ------------------------------------------------------------ as a part: its own tensors and state
    def parts(self):
        return [self, *base.Block.parts(self)]

    def _n(self, i: int) -> str:
        return f"{self.prefix}.{self.names[i]}"

    def weight_specs(self):
        H = self.hidden
        specs = [WeightSpec(self._n(0), (H,), role="norm"), WeightSpec(self._n(2), (H, self.taps), std=0.2), WeightSpec(self._n(4), (self.index + 2,), role="mix")]
        if self.has_ff:
            specs += [WeightSpec(self._n(1), (H,), role="norm"), WeightSpec(self._n(3), (H, self.taps), std=0.2)]
        return specs

    def bind(self, weights, rt):
        # the convolution's taps are stored [channel, tap]; the kernel reads a tap's weights for neighbouring channels together: [tap, channel]
        self.ls1, self.conv1, self.mix = rt.vector(weights[self._n(0)]), rt.vector(weights[self._n(2)].t()), rt.vector(weights[self._n(4)])
        if self.has_ff:
            self.ls2, self.conv2 = rt.vector(weights[self._n(1)]), rt.vector(weights[self._n(3)].t())

    def cache_need(self):
        own = FixedState((2, max(self.taps - 1, 1), self.hidden), torch.float32)   # [sublayer, row, channel]
        return Several((self.mixer.cache_need(), own))

    # ------------------------------------------------------------ one step
    def _layout(self, ctx, state: torch.Tensor, sublayer: int) -> ops.ConvLayout:
        return ops.ConvLayout(self.taps - 1, ctx.seg_of_token, ctx.seg_start, ctx.seg_slot, ctx.n_segments, state[:, sublayer], state.stride(0))

    def _read(self, ctx, norm, x, delta, scale, bias, conv_w, state, sublayer, x_copy=None):
        """The rows a sublayer reads: the contribution before it added to x, the norm, the convolution."""
        layout = self._layout(ctx, state, sublayer)
        h = ctx.rt.empty((ctx.n_tokens, self.hidden))
        if ctx.fixed_shape or ctx.n_segments == ctx.n_tokens:
            # a step of single tokens (decoded tokens): norm and convolution in one kernel, the normed row never leaves the CTA
            ops.add_layernorm_conv_single(x, delta, norm.w, norm.eps, conv_w, h, layout, delta_scale=scale, delta_bias=bias, x_copy=x_copy)
            return h
        ext = norm.forward(ctx, x, delta, delta_scale=scale, delta_bias=bias, x_copy=x_copy, layout=layout)
        ops.causal_conv_rows(ext, conv_w, h, layout)
        return h

    def forward(self, ctx, x, pending, cache):
        if pending is not None:
            raise RuntimeError("this block follows a block that left a contribution to add: mixing arrangements is not supported")
        mixer_cache, own = cache
        state = own.tensor
        key = ("layer results", x.data_ptr())
        stack = ctx.memo.get(key)
        if stack is None:
            stack = ctx.memo[key] = ctx.rt.empty((self.depth + 1, ctx.n_tokens, self.hidden), torch.float32)
        first = stack[0] if self.index == 0 else None       # the embedding's output is the first result; the first norm files it
        h = self._read(ctx, self.mixer_norm, x, None, None, None, self.conv1, state, 0, x_copy=first)
        a = self.mixer.forward(ctx, h, mixer_cache)
        f = None
        if self.has_ff:
            h = self._read(ctx, self.feed_forward_norm, x, a, self.ls1, self.mixer.out_bias, self.conv2, state, 1)
            f = self.feed_forward.forward(ctx, h)
            ops.depth_average(x, f, self.ls2, stack, self.index + 1, self.mix)
        else:
            ops.depth_average(x, a, self.ls1, stack, self.index + 1, self.mix, delta_bias=self.mixer.out_bias)
        return None
