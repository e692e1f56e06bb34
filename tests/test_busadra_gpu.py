"""Busadra in the engine against the plain implementation: each mechanism's kernels alone (with inputs made so that a key just inside
or just outside a window, a far key, a lost state row or a left-out sink shows), then whole models under every way of cutting the
work (in true 32-bit and in bfloat16), pages and slots that are used again, and greedy generation through the engine's entry point
and scheduler."""
from __future__ import annotations

import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_busadra as P
import tiny_busadra as tb
import traces

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOLERANCE = {"float32": 1e-4, "bfloat16": 4e-2}   # of the largest |logit| of the sequence
# bfloat16 only: a router's choice between two experts that score alike may fall the other way after rounding, which changes that
# token's logits (and, through the recurrence, the convolution and attention, later ones) by far more than rounding itself does; with
# random weights and two or three routed layers about one row in fifteen has such a close call. So the bfloat16 comparisons of whole
# models are statistical: the median row is well inside the bound, at most BF16_ROWS_OVER of the rows are beyond it, none is further
# off than BF16_WORST. What has to be exact (windows, state, pages, slots, cuts) is checked in float32, where nothing is allowed.
BF16_ROWS_OVER = 0.12
BF16_MEDIAN = 1e-2
BF16_WORST = 1.5


@pytest.fixture(scope="module")
def bdirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("busadra")
    return {name: tb.write_model(name, root / name) for name in tb.CONFIGS}


@pytest.fixture(scope="module")
def rt32():
    from inference_bench_b200.engine.runtime import Runtime
    return Runtime(DEV, dtype="float32")


@pytest.fixture(scope="module")
def rt16():
    from inference_bench_b200.engine.runtime import Runtime
    return Runtime(DEV, dtype="bfloat16")


def _f32(t):
    return t.to(DEV, torch.float32).contiguous()


def _ctx(rt, runs, slots=None):
    """A step's context for segments given as (first position, tokens); segment i uses row i of whatever table the caller passes on."""
    from inference_bench_b200.engine.context import Segment, build_context
    return build_context(rt, [Segment(i, (slots[i] if slots else i), p0, [0] * n, []) for i, (p0, n) in enumerate(runs)])


# ------------------------------------------------------------------------------------------ norm, convolution, state, depth average
@pytest.mark.parametrize("H,taps", [(80, 3), (132, 1), (256, 5), (4096, 4), (24, 2), (30, 3), (1022, 4)])
def test_layer_norm_convolution_and_its_state_over_portions(rt32, H, taps):
    """Three requests in two slots (one slot is used again, zeroed, by the third) are fed in portions of 1, 2 and more tokens, also
    fewer than taps - 1, together in one batch; every row equals the plain norm and convolution of the whole sequence. The
    contribution added before the norm carries a per-channel scale and a bias."""
    from inference_bench_b200.kernels import ops
    g = torch.Generator().manual_seed(H + taps)
    lens = {"a": 23, "b": 9, "c": 14}
    x = {r: torch.randn((n, H), generator=g) * 3 + 1 for r, n in lens.items()}
    delta = {r: torch.randn((2, n, H), generator=g) for r, n in lens.items()}
    w, scale, bias, cw = torch.rand((H,), generator=g) + 0.5, torch.rand((H,), generator=g), torch.randn((H,), generator=g), torch.randn((H, taps), generator=g) * 0.4
    eps = 1e-5
    want = {}
    for r in lens:
        v = x[r].double() + scale.double() * (delta[r].double().sum(0) + bias.double())
        h = P.layer_norm(v, w, eps)
        want[r] = (v, h + P.causal_conv(h, cw))
    halo = taps - 1
    state = torch.zeros((3, 2, max(halo, 1), H), device=DEV)     # [slots + scratch, sublayer, row, channel]
    state[:, 0] = 7.0                                            # the other sublayer's rows: never touched
    plan = [[("a", 1), ("b", 2)], [("a", 1), ("b", 1)], [("a", 2)], [("a", 7), ("b", 6)], [("c", 1), ("a", 3)], [("c", 2), ("a", 9)], [("c", 11)]]
    slot, at = {"a": 0, "b": 1, "c": 1}, {r: 0 for r in lens}
    for step in plan:
        if step[0][0] == "c" and at["c"] == 0:
            state[1].zero_()                                     # the slot's next request starts from nothing
            state[1, 0] = 7.0
        ctx = _ctx(rt32, [(at[r], n) for r, n in step], [slot[r] for r, _ in step])
        xs = torch.cat([x[r][at[r]:at[r] + n] for r, n in step]).to(DEV).contiguous()
        ds = torch.cat([delta[r][:, at[r]:at[r] + n] for r, n in step], dim=1).to(DEV).contiguous()
        lay = ops.ConvLayout(halo, ctx.seg_of_token, ctx.seg_start, ctx.seg_slot, len(step), state[:, 1], state.stride(0))
        single = None
        if all(n == 1 for _, n in step):   # a step of single tokens: the one-kernel form gives the bits of the two kernels, and the same state
            x1, st1 = xs.clone(), state.clone()
            lay1 = ops.ConvLayout(halo, ctx.seg_of_token, ctx.seg_start, ctx.seg_slot, len(step), st1[:, 1], st1.stride(0))
            single = torch.empty((xs.shape[0], H), device=DEV)
            ops.add_layernorm_conv_single(x1, ds, _f32(w), eps, _f32(cw.t()), single, lay1, delta_scale=_f32(scale), delta_bias=_f32(bias))
            single = (single, x1, st1)
        ext = torch.empty((lay.rows(xs.shape[0]), H), device=DEV)
        ops.add_layernorm(xs, ds, _f32(w), ext, eps, None, _f32(scale), _f32(bias), None, lay)
        for dt, tol in ((torch.float32, 3e-5), (torch.bfloat16, 3e-2)):
            out = torch.empty((xs.shape[0], H), dtype=dt, device=DEV)
            saved = state.clone()
            ops.causal_conv_rows(ext, _f32(cw.t()), out, lay)
            if dt == torch.float32:
                if single is not None:
                    assert torch.equal(single[0], out) and torch.equal(single[1], xs) and torch.equal(single[2], state)
                state.copy_(saved)       # the second pass writes the same state again
            o = 0
            for r, n in step:
                assert torch.allclose(xs[o:o + n].cpu().double(), want[r][0][at[r]:at[r] + n], atol=1e-5, rtol=1e-5)
                err = (out[o:o + n].cpu().double() - want[r][1][at[r]:at[r] + n]).abs().max().item()
                assert err < tol * max(1.0, want[r][1].abs().max().item()), f"request {r} rows {at[r]}..{at[r] + n}: {err}"
                o += n
        for r, n in step:
            at[r] += n
    assert float((state[:, 0] - 7.0).abs().max()) == 0.0
    rt32.check_status()


def test_layer_norm_gathered_rows_and_depth_average(rt32):
    from inference_bench_b200.kernels import ops
    g = torch.Generator().manual_seed(5)
    T, H = 37, 200
    x, w = torch.randn((T, H), generator=g) * 4 - 2, torch.rand((H,), generator=g) + 0.5
    rows = torch.tensor([36, 0, 5, 5], dtype=torch.int32, device=DEV)
    out = torch.empty((4, H), device=DEV)
    xd = _f32(x)
    ops.add_layernorm(xd, None, _f32(w), out, 1e-6, rows)
    assert torch.allclose(out.cpu().double(), P.layer_norm(x.double(), w, 1e-6)[rows.cpu().long()], atol=2e-5)
    assert torch.equal(xd.cpu(), x)
    # depth average: the k-th result is filed and the mix of all results so far goes on
    n = 4
    stack = torch.randn((n + 1, T, H), generator=g)
    for k in (1, 3, 4):
        delta, scale, bias, mix = torch.randn((3, T, H), generator=g), torch.rand((H,), generator=g), torch.randn((H,), generator=g), torch.rand((k + 1,), generator=g)
        sd, xd = _f32(stack), _f32(x)
        ops.depth_average(xd, _f32(delta), _f32(scale), sd, k, _f32(mix), delta_bias=_f32(bias))
        X = x.double() + scale.double() * (delta.double().sum(0) + bias.double())
        want = sum(mix[j].double() * stack[j].double() for j in range(k)) + mix[k].double() * X
        assert torch.allclose(sd[k].cpu().double(), X, atol=1e-5) and torch.allclose(xd.cpu().double(), want, atol=2e-5)
        assert torch.equal(sd[:k].cpu(), stack[:k]) and torch.equal(sd[k + 1:].cpu(), stack[k + 1:])
    v = torch.randn((3, 50), generator=g)
    vd = _f32(v)
    ops.scale_values(vd, 0.37)
    assert torch.allclose(vd.cpu(), v * 0.37)


# ------------------------------------------------------------------------------------------ attention
def _attention_case(dtype, heads, kv_heads, dim, vdim, page, n_ctx, seed=0):
    """Keys and values of one request on shuffled pages of a pool with two layers (the second is used), rows as wide as the larger head."""
    from inference_bench_b200.kernels.ops import KvLayerView
    g = torch.Generator().manual_seed(seed)
    row = max(dim, vdim)
    n_pages = -(-n_ctx // page)
    perm = torch.randperm(n_pages + 3, generator=g)[:n_pages]
    k, v = torch.randn((n_ctx, kv_heads, dim), generator=g), torch.randn((n_ctx, kv_heads, vdim), generator=g)
    pool = torch.zeros((2, n_pages + 3, 2, kv_heads, page, row), dtype=dtype, device=DEV)
    return g, perm, k, v, pool


def _fill(pool, perm, page, k, v):
    for j in range(k.shape[0]):
        pool[1, perm[j // page], 0, :, j % page, :k.shape[2]] = k[j].to(pool.dtype)
        pool[1, perm[j // page], 1, :, j % page, :v.shape[2]] = v[j].to(pool.dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,page,window,cap,sink", [
    (4, 2, 32, 16, 16, 24, 8.0, True), (6, 6, 24, 40, 8, None, 15.0, True), (8, 2, 64, 64, 32, 48, 50.0, True), (4, 1, 128, 128, 16, 17, 10.0, True),
    (6, 6, 64, 64, 16, 96, 20.0, True), (3, 1, 16, 16, 8, 13, None, True), (8, 2, 64, 64, 16, 40, 6.0, False), (8, 8, 64, 64, 64, 64, None, False),
    (8, 2, 64, 64, 16, 40, None, True), (4, 4, 128, 128, 32, None, None, True), (32, 1, 64, 64, 16, 70, 12.0, True)])
def test_attention_windows_far_keys_page_borders_caps_and_the_sink(rt32, rt16, dtype, heads, kv_heads, dim, vdim, page, window, cap, sink):
    """One key is made to stand out for one query (they share a large entry): the last key inside the window and the first outside it,
    the keys on both sides of a page border, a key far back, the query's own position and the one after it; for rows of a prompt
    portion, for the first tokens of a sequence and for decoded tokens. Where the standing-out key is outside, the sink keeps most
    of the weight (the output stays small); scores beyond the cap are capped."""
    from inference_bench_b200.kernels import attention
    rt = rt32 if dtype == torch.float32 else rt16
    n_ctx, scale = 333, 0.2
    g, perm, k, v, pool = _attention_case(dtype, heads, kv_heads, dim, vdim, page, n_ctx, seed=heads * dim + page)
    runs = [(200, 64), (300, 1), (331, 1), (0, 5), (2 * page - 2, 4)]   # (first position, tokens): portions and decoded tokens of the same request
    positions = [p0 + i for p0, n in runs for i in range(n)]
    q = torch.randn((n_ctx, heads, dim), generator=g) * 0.3
    W = window or 10 ** 9
    needles = [(263, 263 - W + 1, 0), (262, 262 - W, 1 % heads), (300, 300 - W + 1, 2 % heads), (331, 331 - W, 0), (331, 332, 1 % heads), (250, 250, 0),
               (2 * page, 2 * page - 1, 0), (2 * page + 1, 2 * page, 1 % heads), (230, 3, 2 % heads), (4, 0, 0)]
    for i, (qp, key, head) in enumerate(needles):
        if not 0 <= key < n_ctx:
            continue
        col = (i * 5) % dim
        k[key, head // (heads // kv_heads), col] = 5.0
        q[qp, head, col] = 30.0
    k, v, q = k.to(dtype).float(), v.to(dtype).float(), q.to(dtype).float()
    _fill(pool, perm, page, k, v)
    want = P.attention_core(q, k, v, scale, cap, window, sink)[positions]
    from inference_bench_b200.kernels.ops import KvLayerView
    ctx = _ctx(rt, runs)
    table = perm.to(torch.int32).reshape(1, -1).repeat(len(runs), 1).contiguous().to(DEV)
    view = KvLayerView(pool, 1, table)
    qd = q[positions].reshape(len(positions), heads * dim).to(DEV, dtype).contiguous()
    plain = not (cap or sink) and dim == vdim
    out = attention.paged_attention(ctx, qd, view, heads, window, scale) if plain else \
        attention.paged_attention(ctx, qd, view, heads, window, scale, qk_dim=dim, v_dim=vdim, softcap=cap or 0.0, sink=sink)
    got = out.float().cpu().double().view(len(positions), heads, vdim)
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    err = (got - want).abs().amax(dim=(1, 2))
    assert err.max().item() < tol, f"positions {[positions[i] for i in torch.nonzero(err >= tol).flatten().tolist()]} differ by up to {err.max().item():.2e}"
    rt.check_status()


@pytest.mark.parametrize("heads,kv_heads,dim,vdim,dims,scaling", [(4, 2, 32, 16, 16, (8.0, 1.0, 4.0, 64)), (6, 6, 24, 40, 8, None), (3, 1, 16, 16, 0, None),
                                                                  (8, 2, 64, 64, 64, (4.0, 1.0, 4.0, 256)), (4, 1, 128, 128, 32, None)])
def test_projection_rows_get_their_bias_and_rotation_and_reach_the_cache(rt32, heads, kv_heads, dim, vdim, dims, scaling):
    """The q/k kernel on partial sums of a [q | k | v] projection whose key and value heads differ in size: biases are added, the first
    `dims` entries of query and key heads are turned by rescaled frequencies, values are not, and keys and values land in their pages."""
    from inference_bench_b200.kernels import ops
    from inference_bench_b200.parts.standard import NoPositionEncoding, RotaryEmbedding
    g = torch.Generator().manual_seed(dim + vdim)
    runs = [(37, 6), (5, 1), (0, 3)]
    ctx = _ctx(rt32, runs)
    T, page, row = 10, 8, max(dim, vdim)
    R = (heads + kv_heads) * dim + kv_heads * vdim
    parts, bias = torch.randn((2, T, R), generator=g), torch.randn((R,), generator=g)
    rope = RotaryEmbedding(dims, 700.0, scaling=scaling) if dims else NoPositionEncoding()
    rope.bind({}, rt32)
    cos, sin = rope.tables(ctx)
    pool = torch.zeros((1, 9, 2, kv_heads, page, row), device=DEV)
    table = torch.tensor([[3, 1, 7, 0, 5, 8], [2, 2, 2, 2, 2, 2], [4, 6, 6, 6, 6, 6]], dtype=torch.int32, device=DEV)
    view = ops.KvLayerView(pool, 0, table)
    qd = torch.empty((T, heads * dim), device=DEV)
    ops.qk_norm_rope_kv(_f32(parts), None, None, 1e-6, cos, sin, ctx.positions, ctx.seg_of_token, qd, view, heads, rt32.status, bias=_f32(bias), qk_dim=dim, v_dim=vdim)
    full = parts.double().sum(0) + bias.double()
    pos = torch.tensor([p0 + i for p0, n in runs for i in range(n)])
    fr = P.rotary_frequencies({"base": 700.0, "dims": dims, "scaling": dict(zip(("factor", "low", "high", "original"), scaling)) if scaling else None}) if dims else torch.zeros(0)
    q = P.rotate(full[:, :heads * dim].view(T, heads, dim), pos, fr)
    kk = P.rotate(full[:, heads * dim:(heads + kv_heads) * dim].view(T, kv_heads, dim), pos, fr)
    vv = full[:, (heads + kv_heads) * dim:].view(T, kv_heads, vdim)
    assert torch.allclose(qd.cpu().double().view(T, heads, dim), q, atol=3e-5)
    seg = ctx.h_seg_of_token
    for t in range(T):
        pg = int(table[seg[t], int(pos[t]) // page])
        assert torch.allclose(pool[0, pg, 0, :, int(pos[t]) % page, :dim].cpu().double(), kk[t], atol=3e-5)
        assert torch.allclose(pool[0, pg, 1, :, int(pos[t]) % page, :vdim].cpu().double(), vv[t], atol=3e-5)
    rt32.check_status()


# ------------------------------------------------------------------------------------------ recurrence
@pytest.mark.parametrize("heads,D,V", [(3, 16, 24), (1, 48, 20), (4, 64, 64), (2, 40, 8), (2, 300, 33), (2, 128, 256), (2, 10, 7), (1, 6, 1)])
def test_recurrence_over_portions_slots_and_long_decoding(rt32, heads, D, V):
    """Two requests advance in one batch in portions of 1, 2, 17 and more tokens (beyond the sixteen the kernel prepares at a time),
    then one of them decodes 150 tokens one by one; a third request takes a freed slot that is zeroed. Gates near 1 for some channels
    (a high floor) keep old tokens in the state, so a lost or stale state shows. Every output equals the plain recurrence over the
    whole sequence, and the state the kernel leaves equals the plain one."""
    from inference_bench_b200.kernels import ops
    g = torch.Generator().manual_seed(D * V)
    lens = {"a": 60 + 150, "b": 41, "c": 20}
    R = heads * (2 * D + V)
    proj = {r: torch.randn((2, n, R), generator=g) for r, n in lens.items()}
    f_bias, lower = torch.randn((heads * D,), generator=g), torch.rand((heads * D,), generator=g) * 0.9
    lower[::3] = 0.995
    want, want_state = {}, {}
    for r, n in lens.items():
        z = proj[r].double().sum(0)
        q = P.silu(z[:, :heads * D]).view(n, heads, D)
        lo = lower.double().view(heads, D)
        f = lo + (1 - lo) * torch.sigmoid(z[:, heads * D:2 * heads * D] + f_bias.double()).view(n, heads, D)
        want[r], want_state[r] = P.recurrence_core(q, f, z[:, 2 * heads * D:].view(n, heads, V))
    state = torch.zeros((3, heads, D, V), device=DEV)
    plan = [[("a", 1), ("b", 2)], [("a", 2), ("b", 17)], [("b", 22), ("a", 40)], [("c", 3), ("a", 17)], [("c", 17)]] + [[("a", 1)]] * 150
    slot, at = {"a": 0, "b": 1, "c": 1}, {r: 0 for r in lens}
    worst = 0.0
    # the chunked form of long segments: both requests whole in one step (210 and 41 rows: one goes in chunks, the other token by token), then
    # a second long portion on top of a state that is not zero
    for step in ([("a", 210), ("b", 41)], [("a", 70), ("b", 2)], [("a", 140), ("b", 39)]):
        if step[0][1] != 140:
            st2 = torch.zeros((3, heads, D, V), device=DEV)
            at2 = {r: 0 for r in lens}
        from inference_bench_b200.parts.recurrent import GatedLinearRecurrence
        ctx = _ctx(rt32, [(at2[r], n) for r, n in step], [slot[r] for r, _ in step])
        short, long_segs, chunks = GatedLinearRecurrence._cut(ctx)
        assert long_segs is not None and long_segs.shape[0] == 1 and short.tolist() == [1]
        pr = torch.cat([proj[r][:, at2[r]:at2[r] + n] for r, n in step], dim=1).to(DEV).contiguous()
        o = torch.empty((pr.shape[1], heads, V), device=DEV)
        ops.gated_recurrence(pr, _f32(f_bias), _f32(lower), st2, ctx.seg_start, ctx.seg_slot, len(step), o, heads, D, V, seg_list=short, long_segs=long_segs, chunks=chunks)
        k = 0
        for r, n in step:
            err = (o[k:k + n].cpu().double() - want[r][at2[r]:at2[r] + n]).abs().max().item()
            assert err < 2e-4 * max(1.0, want[r].abs().max().item()), f"chunked form, request {r} rows {at2[r]}..{at2[r] + n}: {err}"
            k, at2[r] = k + n, at2[r] + n
        if at2["a"] == 210:
            assert torch.allclose(st2[0].cpu().double(), want_state["a"], atol=1e-4) and torch.allclose(st2[1].cpu().double(), want_state["b"], atol=1e-4)
    for step in plan:
        if step[0][0] == "c" and at["c"] == 0:
            assert torch.allclose(state[1].cpu().double(), want_state["b"], atol=1e-4)
            state[1].zero_()
        ctx = _ctx(rt32, [(at[r], n) for r, n in step], [slot[r] for r, _ in step])
        pr = torch.cat([proj[r][:, at[r]:at[r] + n] for r, n in step], dim=1).to(DEV).contiguous()
        T = pr.shape[1]
        o = torch.empty((T, heads, V), device=DEV)
        ops.gated_recurrence(pr, _f32(f_bias), _f32(lower), state, ctx.seg_start, ctx.seg_slot, len(step), o, heads, D, V)
        k = 0
        for r, n in step:
            worst = max(worst, (o[k:k + n].cpu().double() - want[r][at[r]:at[r] + n]).abs().max().item())
            k, at[r] = k + n, at[r] + n
    assert at == lens and worst < 2e-4 * max(1.0, max(w.abs().max().item() for w in want.values())), worst
    assert torch.allclose(state[0].cpu().double(), want_state["a"], atol=1e-4)
    # the per-head norm that follows
    w = torch.rand((V,), generator=g) + 0.5
    o = want["b"].float()
    for dt, tol in ((torch.float32, 2e-5), (torch.bfloat16, 2e-2)):
        out = torch.empty((o.shape[0], heads * V), dtype=dt, device=DEV)
        ops.head_rmsnorm(_f32(o), _f32(w), 1e-5, out)
        assert torch.allclose(out.cpu().double().view(-1, heads, V), P.rms_unit(o.double(), 1e-5) * w.double(), atol=tol, rtol=tol)


# ------------------------------------------------------------------------------------------ experts
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("W,ff,E,top,T", [(80, 24, 5, 2, 37), (132, 36, 7, 1, 9), (256, 64, 16, 4, 300), (64, 128, 4, 4, 1)])
def test_experts_chosen_by_sigmoid_scores_with_the_weight_on_their_input(rt32, rt16, dtype, W, ff, E, top, T):
    """The part alone: the router's sigmoid scores choose, the weights are the scores themselves (not renormalised: they do not sum to
    one) and scale what the expert reads. A weight on the output instead would differ by far more than the tolerance."""
    from inference_bench_b200.engine.context import StepContext
    from inference_bench_b200.parts.experts import RoutedExperts
    rt = rt32 if dtype == "float32" else rt16
    g = torch.Generator().manual_seed(W + T)
    w = {"m.router": (torch.randn((E, W), generator=g) * 2 / W ** 0.5).to(torch.bfloat16)}
    for k in range(E):
        w[f"m.e{k}.gate"], w[f"m.e{k}.up"] = [(torch.randn((ff, W), generator=g) * 2 / W ** 0.5).to(torch.bfloat16) for _ in range(2)]
        w[f"m.e{k}.down"] = (torch.randn((W, ff), generator=g) / ff ** 0.5).to(torch.bfloat16)
    h = torch.randn((T, W), generator=g).to(torch.bfloat16)
    f = {"router": {"experts": E, "top": top}}
    want = P.experts(h.double(), f, w, "m")
    idx, wt = P.route(h.double(), f, w, "m")
    wrong = torch.zeros_like(want)
    for t in range(T):
        for e, c in zip(idx[t].tolist(), wt[t].tolist()):
            wrong[t] += c * (w[f"m.e{e}.down"].double() @ (P.silu(w[f"m.e{e}.gate"].double() @ h[t].double()) * (w[f"m.e{e}.up"].double() @ h[t].double())))
    part = RoutedExperts("m", W, ff, E, top, score="sigmoid", weight_on="input")
    part.bind({n: t.to(DEV) for n, t in w.items()}, rt)
    ctx = _ctx(rt, [(0, T)])
    out = part.forward(ctx, h.to(DEV, rt.act_dtype).contiguous()).sum(0).cpu().double()
    scale = want.abs().max().item()
    tol = 2e-5 if dtype == "float32" else 3e-2
    err = (out - want).abs().amax(dim=1) / scale
    if top < E:   # rows whose choice rests on a close call may fall the other way in bfloat16
        close = (torch.sigmoid(h.double() @ w["m.router"].double().T).topk(top + 1).values[:, top - 1:top + 1].diff().abs().flatten() < 2e-2)
        err = err[~close] if dtype == "bfloat16" else err
    assert err.numel() == 0 or err.max().item() < tol, err.max().item()
    assert ((wrong - want).abs().max() / scale).item() > 0.1
    rt.check_status()


# ------------------------------------------------------------------------------------------ whole models
def _requests(name):
    vocab = tb.CONFIGS[name]["config"]["vocab"]
    return {r: traces.prompt(300 + i, n, vocab) for i, (r, n) in enumerate({"a": 150, "b": 1, "c": 23, "d": 64, "e": 97, "f": 2}.items())}


@pytest.fixture(scope="module")
def plain_logits(bdirs):
    return {name: {r: P.PlainBusadra(bdirs[name]).logits(t).numpy() for r, t in _requests(name).items()} for name in tb.CONFIGS}


def _runner(bdirs, name, dtype, max_tokens, **kw):
    from inference_bench_b200.trace import build_runner
    return build_runner(bdirs[name], dtype, max_tokens, page_size=tb.CONFIGS[name]["page_size"], **kw)


def _compare(got, want_by_req, dtype, what):
    worst, over, errs = 0.0, 0, []
    for (r, pos), row in got.items():
        want = want_by_req[r][pos]
        err = np.abs(row - want).max() / np.abs(want_by_req[r]).max()
        if dtype == "bfloat16" and TOLERANCE[dtype] < err <= BF16_WORST:
            over += 1
        else:
            assert err <= TOLERANCE[dtype], f"{what}: request {r} position {pos}: |diff| = {err:.3e} of max|logit| (allowed {TOLERANCE[dtype]:.0e})"
        worst = max(worst, err)
        errs.append(err)
    assert len(got) == sum(len(v) for v in want_by_req.values())
    allowed = max(BF16_ROWS_OVER * len(got), 3) if dtype == "bfloat16" else 0
    assert over <= allowed, f"{what}: {over} of {len(got)} rows are beyond {TOLERANCE[dtype]:.0e} of max|logit| (allowed {allowed:.0f})"
    if dtype == "bfloat16":
        assert float(np.median(errs)) < BF16_MEDIAN, f"{what}: the median row differs by {np.median(errs):.2e} of max|logit|"
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tb.CONFIGS))
def test_layers_one_by_one(bdirs, name, dtype):
    """The residual stream after every layer against the plain model's, so that a wrong layer is named."""
    from inference_bench_b200.engine.step import StepEntry
    toks = _requests(name)["e"]
    want = P.PlainBusadra(bdirs[name]).hidden_states(toks)
    runner = _runner(bdirs, name, dtype, 128)
    runner.cache.admit("x")
    layers = []
    runner.step([StepEntry("x", toks, list(range(len(toks))))], trace=layers)
    assert len(layers) == len(want)
    for i, (g, w) in enumerate(zip(layers, want)):
        err = (g.cpu().double() - w).abs().amax(dim=1) / w.abs().max().item()
        where = f"{name}/{dtype}: the stream after {'the embedding' if i == 0 else f'layer {i - 1}'}"
        if dtype == "float32":
            assert err.max().item() < 2e-5, f"{where} differs by {err.max().item():.2e}"
        else:
            assert err.median().item() < BF16_MEDIAN and (err > 4e-2).sum().item() <= max(3, BF16_ROWS_OVER * len(toks)) and err.max().item() < BF16_WORST, \
                f"{where} differs by {err.max().item():.2e} (median {err.median().item():.2e})"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tb.CONFIGS))
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
def test_cut_matches_plain(bdirs, plain_logits, name, dtype, cut):
    """Whole prompts; prompts then the last tokens one by one (a tail long enough for every window to pass over decoded tokens only);
    portions down to two tokens; up to four live requests of unequal length in one batch with a pool that only holds what is live, so
    pages and slots are used again by later requests."""
    reqs = _requests(name)
    steps = {"whole": traces.whole, "tail": lambda r: traces.tail_one_by_one(r, tail=60), "portions": traces.portions, "mixed": traces.mixed}[cut](reqs)
    max_tokens = traces.max_live_tokens(steps)
    runner = _runner(bdirs, name, dtype, max_tokens, max_requests=4)
    got = traces.run_steps(runner, steps)
    worst = _compare(got, plain_logits[name], dtype, f"{name}/{dtype}/{cut}")
    runner.cache.check()
    assert runner.cache.used_pages() == [0] * len(runner.cache.groups)
    print(f"{name}/{dtype}/{cut}: worst {worst:.3e} of max|logit|, pool {max_tokens} tokens")


def test_a_request_alone_and_in_a_batch_give_the_same_float32_logits(bdirs):
    """The float32 path adds in one order whatever shares the step: a request beside three others of other lengths, on other pages
    and in another slot, gives the bits it gives alone."""
    from inference_bench_b200.engine.step import StepEntry
    name = "A"
    reqs = _requests(name)
    runner = _runner(bdirs, name, "float32", 1024, max_requests=4)
    runner.cache.admit("alone")
    alone = runner.step([StepEntry("alone", reqs["d"], [len(reqs["d"]) - 1])]).cpu()
    runner.cache.release("alone")
    for r in ("c", "f", "d", "a"):
        runner.cache.admit(r)
    rows = runner.step([StepEntry(r, reqs[r], [len(reqs[r]) - 1]) for r in ("c", "f", "d", "a")]).cpu()
    assert torch.equal(rows[2], alone[0])


@pytest.mark.parametrize("name", list(tb.CONFIGS))
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_engine(bdirs, name, graphs):
    """`Engine.generate`: the scheduler cuts prompts into portions, batches them beside decoded tokens, and decode steps run as
    captured graphs or not; float32 tokens equal the plain model's."""
    from inference_bench_b200 import Engine
    vocab = tb.CONFIGS[name]["config"]["vocab"]
    plain = P.PlainBusadra(bdirs[name])
    prompts = [traces.prompt(70 + i, n, vocab) for i, n in enumerate((5, 21, 40))]
    want = [plain.greedy(p, 7) for p in prompts]
    eng = Engine(bdirs[name], dtype="float32", max_ctx=128, page_size=tb.CONFIGS[name]["page_size"], use_graphs=graphs, prefill_chunk=9, max_batched_tokens=16)
    got = eng.generate(prompts, max_tokens=7)
    assert [r.tokens for r in got] == want
    assert eng.cache.used_pages() == [0] * len(eng.cache.groups)
    eng.cache.check()
    one = eng.generate(prompts[1], max_tokens=7)
    assert one.tokens == want[1]


def test_generation_in_bfloat16_runs_and_long_decoding_stays_close(bdirs):
    from inference_bench_b200 import Engine
    name = "C"
    vocab = tb.CONFIGS[name]["config"]["vocab"]
    plain = P.PlainBusadra(bdirs[name])
    prompt = traces.prompt(5, 12, vocab)
    eng = Engine(bdirs[name], dtype="bfloat16", max_ctx=256, page_size=32)
    got = eng.generate(prompt, max_tokens=120).tokens
    assert len(got) == 120
    lg = plain.logits(prompt + got)     # teacher-forced on the engine's own tokens, the plain model ranks every chosen token near the top
    span = float(lg.max() - lg.min())
    below = [float(lg[len(prompt) + i - 1].max() - lg[len(prompt) + i - 1][tok]) / span for i, tok in enumerate(got)]
    assert all(math.isfinite(b) for b in below) and max(below) < 0.5
    assert sum(b > 0.05 for b in below) <= BF16_ROWS_OVER * len(got), f"{sum(b > 0.05 for b in below)} decoded tokens lie more than 5 % of the logits' span below the plain model's best"


def test_trace_replay_program_and_command_line(bdirs, tmp_path):
    """bin/trace_run as a subprocess fed JSON steps (a mixed trace, float32), and `run` and `spec` of the command line, on a model
    folder of this architecture: nothing in them names an architecture."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    name = "A"
    vocab = tb.CONFIGS[name]["config"]["vocab"]
    reqs = {r: traces.prompt(900 + i, n, vocab) for i, (r, n) in enumerate({"a": 70, "b": 9, "c": 33, "d": 64, "e": 2}.items())}
    steps = traces.mixed(reqs, seed=5)
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(bdirs[name]), "--dtype", "float32", "--out", str(out),
                           "--max-tokens", str(traces.max_live_tokens(steps))],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    plain = P.PlainBusadra(bdirs[name])
    want = {r: plain.logits(t).numpy() for r, t in reqs.items()}
    at = {r: 0 for r in reqs}
    for s in steps:
        rows = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab)
        k = 0
        for e in s["entries"]:
            for w in e["want"]:
                err = np.abs(rows[k] - want[e["id"]][at[e["id"]] + w]).max() / np.abs(want[e["id"]]).max()
                assert err <= TOLERANCE["float32"]
                k += 1
            at[e["id"]] += len(e["tokens"])
        assert k == rows.shape[0]
    env = dict(os.environ, PYTHONPATH=root)
    p = subprocess.run([sys.executable, "-m", "inference_bench_b200", "run", "--model", str(bdirs[name]), "--prompt-len", "12", "--max-tokens", "5", "--json",
                        "--dtype", "float32", "--max-ctx", "64"], capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    r = json.loads(p.stdout)
    from inference_bench_b200.cli import _synthetic_prompt
    assert r["prompt_tokens"] == 12 and r["tokens"] == plain.greedy(_synthetic_prompt(12, vocab), 5)
    p = subprocess.run([sys.executable, "-m", "inference_bench_b200", "spec", "--model", str(bdirs[name])], capture_output=True, text=True, env=env)
    assert p.returncode == 0 and json.loads(p.stdout)["layers"][1]["mixer"]["mask"]["size"] == 24
