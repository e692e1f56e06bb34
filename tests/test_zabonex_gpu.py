"""Zabonex in the engine against the plain implementation: each mechanism's kernels alone, then whole models under every way
of cutting the work (in true 32-bit and in bfloat16), pages and slots that are used again, and greedy generation through the
engine's entry point and scheduler."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import plain_zabonex as P
import tiny_zabonex as tz
import traces

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOLERANCE = {"float32": 1e-4, "bfloat16": 4e-2}   # of the largest |logit| of the sequence
# bfloat16 only: a router's choice between two experts (or groups) that score alike may fall the other way after rounding, which
# changes that token's logits by far more than rounding itself does; a model that sends a token to one expert of one group is
# full of such tokens. So a few rows may exceed the bound: 4 % of them, or half as many again as exceed it when the plain model
# itself rounds to bfloat16 where a 16-bit implementation may (plain_zabonex.bf16), and none may be further off than there.
BF16_ROWS_OVER = 0.04
BF16_WORST = 0.5


@pytest.fixture(scope="module")
def zdirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("zabonex")
    return {name: tz.write_model(name, root / name) for name in tz.CONFIGS}


@pytest.fixture(scope="module")
def rt32():
    from inference_bench_b200.engine.runtime import Runtime
    return Runtime(DEV, dtype="float32")


def _f32(t):
    return t.to(DEV, torch.float32).contiguous()


# ------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("T,H,P_", [(1, 80, 1), (5, 132, 3), (300, 192, 2), (3, 4096, 1)])
def test_norm_on_a_sublayer_output(rt32, T, H, P_):
    from inference_bench_b200.kernels import ops
    g = torch.Generator().manual_seed(T * H)
    x, delta, w = torch.randn((T, H), generator=g), torch.randn((P_, T, H), generator=g) * 3, torch.rand((H,), generator=g) * 0.6 - 0.3
    for mult, eps in ((1.0, 1e-6), (0.35, 1e-2)):
        want = x.double() + mult * P.norm_offset(delta.double().sum(0), w.double(), eps)
        xd, act = _f32(x), torch.empty((T, H), dtype=torch.bfloat16, device=DEV)
        ops.norm_residual(xd, _f32(delta), _f32(w) + 1.0, mult, eps, act)
        assert torch.allclose(xd.cpu().double(), want, atol=2e-5, rtol=1e-5)
        assert torch.equal(act.cpu(), xd.cpu().to(torch.bfloat16))


def _latent_case(rt, dtype, H, rank, rot, page, ctx_len, rows, seed=0):
    """A cache of `ctx_len` rows for one request on shuffled pages, and queries [len(rows), H, rank + rot] at positions `rows`."""
    from inference_bench_b200.kernels.ops import KvLayerView
    g = torch.Generator().manual_seed(seed)
    D = rank + rot
    n_pages = -(-ctx_len // page)
    perm = torch.randperm(n_pages + 3, generator=g)[:n_pages]
    cache = torch.randn((ctx_len, D), generator=g)
    pool = torch.zeros((2, n_pages + 3, 1, 1, page, D), dtype=dtype, device=DEV)
    for j in range(ctx_len):
        pool[1, perm[j // page], 0, 0, j % page] = cache[j].to(dtype)
    table = perm.to(torch.int32).reshape(1, -1).to(DEV)
    q = torch.randn((len(rows), H, D), generator=g) * 0.3
    view = KvLayerView(pool, 1, table)
    return cache.to(dtype).double(), q, view


def _plain_latent_rows(cache, q, positions, rank, scale):
    out = torch.zeros((q.shape[0], q.shape[1], rank), dtype=torch.float64)
    for i, p in enumerate(positions):
        s = (q[i].double() @ cache[:p + 1].T) * scale
        out[i] = torch.softmax(s, dim=-1) @ cache[:p + 1, :rank]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,rank,rot,page", [(3, 40, 8, 16), (11, 72, 12, 8), (16, 128, 16, 32), (8, 300, 2, 16), (5, 64, 32, 16), (40, 512, 64, 64), (16, 48, 16, 8)])
def test_latent_attention_kernel_far_keys_page_borders_and_the_causal_edge(rt32, dtype, H, rank, rot, page):
    """One key is made to stand out for one head (its latent and the query share a large entry): the key far back, the keys on both
    sides of a page border, the query's own position (the last key it sees) and the one after it (which it must not see), for a
    token of a prompt portion and for a decoded token whose keys are cut into slices."""
    from inference_bench_b200.kernels import ops
    ctx_len, scale = 333, 0.21
    rows = [0, 1, page - 1, page, page + 1, 200, 300, 300, 331, 331]   # positions of the queries
    cache, q, view = _latent_case(rt32, dtype, H, rank, rot, page, ctx_len, rows)
    pool = view.pool
    needles = {5: (3, 0), 6: (2 * page - 1, 1 % H), 7: (2 * page, 2 % H), 8: (331, 0), 9: (332, 1 % H)}   # query row -> (key, head)
    for r, (key, head) in needles.items():
        col = (r * 7) % rank
        cache[key, col] = 6.0
        page_id = int(view.block_table[0, key // page])
        pool[1, page_id, 0, 0, key % page, col] = 6.0
        q[r, head, col] = 40.0
    want = _plain_latent_rows(cache, q, rows, rank, scale)
    # the needle rows really rest on their key: nearly all weight where the key is visible, none where it is not
    assert abs(want[5, 0, (5 * 7) % rank].item() - 6.0) < 0.05 and abs(want[9, 1 % H, (9 * 7) % rank].item()) < 4.5
    T = len(rows)
    pos = torch.tensor(rows, dtype=torch.int32, device=DEV)
    seg = torch.zeros(T, dtype=torch.int32, device=DEV)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for n_slices, slice_keys in ((1, 1 << 30), (6, 64), (11, 32)):
        out = torch.empty((T, H, rank), dtype=dtype, device=DEV)
        scratch = (torch.empty(T * H * n_slices * rank, device=DEV), torch.empty(T * H * n_slices * 2, device=DEV))
        ops.latent_attention(_f32(q), view, pos, seg, scale, out, rank, n_slices, slice_keys, scratch, rt32.status)
        err = (out.cpu().double() - want).abs().max().item()
        assert err < tol, f"{n_slices} slices: {err}"
        if dtype == torch.bfloat16 and ops.latent_attention_mma_supports(rank, rank + rot) and slice_keys % 64 == 0:
            # the tensor-core kernel rounds the queries to bfloat16 too: compare with the plain sum over those
            want16 = _plain_latent_rows(cache, q.to(torch.bfloat16).float(), rows, rank, scale)
            for cta_rows in (16, 32, 64):   # query rows a CTA holds: the heads of one token, or of several consecutive tokens
                if cta_rows > ops.latent_attention_mma_rows(rank, rank + rot, 64):
                    continue
                per = max(1, cta_rows // H)
                for units in ([None] if per == 1 else [None, torch.tensor([(t, min(per, T - t)) for t in range(0, T, per)], dtype=torch.int32, device=DEV)]):
                    out = torch.full((T, H, rank), 9.0, dtype=dtype, device=DEV)
                    ops.latent_attention_mma(_f32(q), view, pos, seg, units, scale, out, rank, n_slices, slice_keys, scratch, rt32.status, cta_rows)
                    err = (out.cpu().double() - want16).abs().max().item()
                    assert err < 3e-2, f"tensor cores, {cta_rows} rows a CTA, {n_slices} slices, {'a CTA per token' if units is None else 'tokens sharing a CTA'}: {err}"
    rt32.check_status()


@pytest.mark.parametrize("H,dim,rot,rank,dims", [(3, 24, 8, 40, 8), (11, 16, 12, 72, 6), (2, 5, 0, 33, 0)])
def test_latent_prepare_writes_queries_and_the_cache_row(rt32, H, dim, rot, rank, dims):
    """The fused projection's partial sums -> unrotated query parts, rotated query parts, and the normed latent with the rotated key
    part in the cache, at positions up to a few thousand (angles in 32-bit) and in pages that are not in order."""
    from inference_bench_b200.kernels import ops
    from inference_bench_b200.kernels.ops import KvLayerView
    g = torch.Generator().manual_seed(H)
    T, page, base, eps, Pn = 6, 8, 5000.0, 1e-5, 3
    positions = [0, 1, 7, 8, 1000, 3001]
    R = H * (dim + rot) + rank + rot
    qd = torch.randn((Pn, T, R), generator=g)
    cw = torch.rand((rank,), generator=g) + 0.5
    n_pages = 3001 // page + 1
    pool = torch.zeros((1, n_pages, 1, 1, page, rank + rot), device=DEV)
    table = torch.arange(n_pages, dtype=torch.int32).flip(0).reshape(1, -1).contiguous().to(DEV)
    view = KvLayerView(pool, 0, table)
    pos = torch.tensor(positions, dtype=torch.int32, device=DEV)
    cos = sin = None
    if dims:
        i = torch.arange(dims // 2, dtype=torch.float64)
        ang = (torch.tensor(positions, dtype=torch.float64)[:, None] * base ** (-2.0 * i / dims)[None]).float()
        cos, sin = _f32(torch.cos(ang)), _f32(torch.sin(ang))
    q_nope = torch.empty((T, H, dim), device=DEV)
    q_full = torch.zeros((T, H, rank + rot), device=DEV)
    ops.latent_prepare(_f32(qd), _f32(cw), eps, cos, sin, pos, torch.zeros(T, dtype=torch.int32, device=DEV), q_nope, q_full, view, H, dim, rot, rank, True, rt32.status)
    s = qd.double().sum(0)
    q = s[:, :H * (dim + rot)].view(T, H, dim + rot)
    assert torch.allclose(q_nope.cpu().double(), q[..., :dim], atol=1e-5)
    qr = P.rotate_pairs(q[..., dim:].transpose(0, 1), torch.tensor(positions), base, dims).transpose(0, 1) if dims else q[..., dim:]
    assert torch.allclose(q_full.cpu().double()[..., rank:], qr, atol=2e-3 if max(positions) > 100 else 1e-5)   # float32 angles at position 3001
    c = P.norm_plain(s[:, H * (dim + rot):H * (dim + rot) + rank], cw.double(), eps)
    kr = s[:, H * (dim + rot) + rank:]
    kr = P.rotate_pairs(kr, torch.tensor(positions), base, dims) if dims else kr
    for t, p in enumerate(positions):
        row = pool[0, n_pages - 1 - p // page, 0, 0, p % page].cpu().double()
        assert torch.allclose(row[:rank], c[t], atol=1e-5) and torch.allclose(row[rank:], kr[t], atol=2e-3)
    rt32.check_status()


def test_per_head_products(rt32):
    from inference_bench_b200.kernels import ops
    g = torch.Generator().manual_seed(3)
    for T, H, N, K, pad in ((1, 3, 40, 24, 8), (70, 11, 10, 72, 0), (130, 2, 65, 17, 3), (200, 4, 130, 136, 6)):
        x, w = torch.randn((T, H, K), generator=g), torch.randn((H, N, K), generator=g)
        out = torch.full((T, H, N + pad), 7.0, device=DEV)
        ops.gemm_heads(_f32(x), _f32(w), out, N)
        want = torch.einsum("thk,hnk->thn", x.double(), w.double())
        assert torch.allclose(out.cpu().double()[..., :N], want, atol=1e-4)
        assert (out[..., N:] == 7.0).all()
        if K % 8 == 0:   # bfloat16 operands on the tensor cores, float32 and bfloat16 outputs
            xb, wb = x.to(DEV, torch.bfloat16), w.to(DEV, torch.bfloat16)
            want16 = torch.einsum("thk,hnk->thn", xb.cpu().double(), wb.cpu().double())
            for dt, atol, rtol in ((torch.float32, 1e-4, 1e-5), (torch.bfloat16, 1e-2, 1e-2)):
                out = torch.full((T, H, N + pad), 7.0, device=DEV, dtype=dt)
                ops.gemm_heads(xb, wb, out, N, tensor_cores=True)
                assert torch.allclose(out.cpu().double()[..., :N], want16, atol=atol, rtol=rtol) and (out[..., N:] == 7.0).all()


@pytest.mark.parametrize("E,groups,keep,top,scale", [(12, 4, 2, 3, 2.0), (64, 8, 3, 6, 0.5), (5, 1, 1, 1, 1.0), (6, 3, 1, 2, 1.0), (40, 40, 7, 7, 1.0)])
def test_router_choice(rt32, E, groups, keep, top, scale):
    from inference_bench_b200.kernels import ops
    g = torch.Generator().manual_seed(E)
    T, Pn = 97, 2
    logits = torch.randn((Pn, T, E), generator=g) * 2
    # token 1: the two best experts lie in the first group and the third best in the last: where one group stays, the third best
    # must not be chosen although it beats every other expert of the first group
    logits[:, 1] = -3.0 + torch.arange(E) * 0.01   # no two alike: no choice rests on a tie
    logits[:, 1, 0] = 2.0
    logits[:, 1, 1] = 1.9
    logits[:, 1, E - 1] = 1.5
    r = {"experts": E, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}}
    want_idx, want_wt = P.route(logits.double().sum(0), torch.eye(E, dtype=torch.float64), r)   # the logits themselves as the router's input
    idx = torch.empty((T, top), dtype=torch.int32, device=DEV)
    wt = torch.empty((T, top), device=DEV)
    ops.moe_route(_f32(logits), groups, keep, top, scale, False, idx, wt)
    assert torch.equal(idx.cpu().long().sort(dim=1).values, want_idx.sort(dim=1).values)
    got = torch.zeros((T, E), dtype=torch.float64).scatter_(1, idx.cpu().long(), wt.cpu().double())
    want = torch.zeros((T, E), dtype=torch.float64).scatter_(1, want_idx, want_wt)
    assert torch.allclose(got, want, atol=1e-6)
    if groups > 1 and keep == 1 and E // groups < E - 1 and top >= 2:
        assert E - 1 not in idx[1].tolist()


@pytest.mark.parametrize("T", [1, 2, 9, 150])
@pytest.mark.parametrize("E,top,W,F", [(5, 1, 80, 40), (16, 4, 132, 36), (3, 3, 64, 70), (7, 2, 200, 136), (6, 2, 136, 192)])
def test_experts_on_regrouped_rows(rt32, T, E, top, W, F):
    """Regrouping by expert, the experts' two products and the weighted sum, against the plain loop over tokens; the rows an expert
    gets span several tiles for the largest T and some experts get none for the smallest."""
    from inference_bench_b200.kernels import ops
    g = torch.Generator().manual_seed(T + E)
    h = torch.randn((T, W), generator=g)
    w_gu = torch.randn((E, 2 * F, W), generator=g) / W ** 0.5
    w_d = torch.randn((E, W, F), generator=g) / F ** 0.5
    idx = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    wt = torch.rand((T, top), generator=g)
    base = torch.randn((2, T, W), generator=g)
    want = base.double().sum(0)
    for t in range(T):
        for k in range(top):
            e = int(idx[t, k])
            want[t] += wt[t, k].double() * P.gated_ff(h[t:t + 1].double(), w_gu[e, :F].double(), w_gu[e, F:].double(), w_d[e].double())[0]
    R = T * top
    d = lambda n: torch.empty((n,), dtype=torch.int32, device=DEV)
    offsets, tile_start, row_of_pair, token_of_row = d(E + 1), d(E + 1), d(R), d(R)
    idx_d = idx.to(DEV)
    ops.moe_sort(idx_d, E, offsets, tile_start, row_of_pair, token_of_row)
    counts = torch.bincount(idx.flatten().long(), minlength=E)
    assert offsets.cpu().tolist() == [0] + counts.cumsum(0).tolist()
    assert sorted(row_of_pair.cpu().tolist()) == list(range(R))
    assert torch.equal(token_of_row.cpu()[row_of_pair.cpu().long()], torch.arange(R, dtype=torch.int32) // top)
    act, y, out = torch.empty((R, F), device=DEV), torch.empty((R, W), device=DEV), torch.empty((T, W), device=DEV)
    ops.gemm_grouped(_f32(h), token_of_row, _f32(w_gu), act, offsets, tile_start, gated=True)
    ops.gemm_grouped(act, None, _f32(w_d), y, offsets, tile_start, gated=False)
    ops.moe_combine(y, row_of_pair, _f32(wt), _f32(base), out)
    assert torch.allclose(out.cpu().double(), want, atol=1e-4)
    if W % 8 == 0 and F % 8 == 0:   # the same on the tensor cores with bfloat16 operands (the activation handed on in bfloat16)
        hb, gub, db = h.to(DEV, torch.bfloat16), w_gu.to(DEV, torch.bfloat16), w_d.to(DEV, torch.bfloat16)
        want16 = base.double().sum(0)
        for t in range(T):
            for k in range(top):
                e = int(idx[t, k])
                want16[t] += wt[t, k].double() * P.gated_ff(hb[t:t + 1].cpu().double(), gub[e, :F].cpu().double(), gub[e, F:].cpu().double(), db[e].cpu().double(), P.bf16)[0]
        act16 = torch.empty((R, F), device=DEV, dtype=torch.bfloat16)
        ops.gemm_grouped(hb, token_of_row, gub, act16, offsets, tile_start, gated=True, tensor_cores=True)
        ops.gemm_grouped(act16, None, db, y, offsets, tile_start, gated=False, tensor_cores=True)
        ops.moe_combine(y, row_of_pair, _f32(wt), _f32(base), out)
        assert torch.allclose(out.cpu().double(), want16, atol=2e-3)
        # and on tcgen05: the rows gathered into the experts' order first, token tiles of every size the kernel has
        from inference_bench_b200.kernels import gemm_tcgen05 as G
        for bn in (16, 32, 64, 128, 256):
            if not G.grouped_supported(W, F, bn):
                continue
            ops.moe_sort(idx_d, E, offsets, tile_start, row_of_pair, token_of_row, tile_rows=bn)
            xs = torch.empty((R, W), device=DEV, dtype=torch.bfloat16)
            ops.gather_rows(hb, token_of_row, xs)
            assert torch.equal(xs, hb[token_of_row.long()])
            act16.fill_(7.0), y.fill_(7.0)
            G.gemm_grouped_swiglu(xs, gub, act16, bn, offsets, tile_start, rt32.status)
            G.gemm_grouped(act16, db, y, bn, offsets, tile_start, rt32.status)
            ops.moe_combine(y, row_of_pair, _f32(wt), _f32(base), out)
            assert torch.allclose(out.cpu().double(), want16, atol=3e-3), f"token tile {bn}"
        rt32.check_status()


# ------------------------------------------------------------------------------------------ whole models
LENGTHS = {"a": 7, "b": 19, "c": 33, "d": 70, "e": 45, "f": 130, "g": 2, "h": 64, "i": 1}


def _requests(name):
    vocab = tz.CONFIGS[name]["config"]["vocab"]
    return {r: traces.prompt(300 + i, n, vocab) for i, (r, n) in enumerate(LENGTHS.items())}


@pytest.fixture(scope="module")
def plain_logits(zdirs):
    out = {}
    for name in tz.CONFIGS:
        m = P.PlainZabonex(zdirs[name])
        out[name] = {r: m.logits(t).numpy() for r, t in _requests(name).items()}
        over, worst = 0, 0.0
        for r, t in _requests(name).items():
            err = np.abs(m.logits(t, P.bf16).numpy() - out[name][r]).max(axis=1) / np.abs(out[name][r]).max()
            over, worst = over + int((err > TOLERANCE["bfloat16"]).sum()), max(worst, float(err.max()))
        ROUNDED[name] = (over, worst)
    return out


ROUNDED: dict = {}   # per configuration: (rows beyond the bfloat16 bound, worst row) of the plain model with bfloat16 rounding


def _runner(zdirs, name, dtype, max_tokens, **kw):
    from inference_bench_b200.trace import build_runner
    return build_runner(zdirs[name], dtype, max_tokens, page_size=tz.CONFIGS[name]["page_size"], **kw)


def _compare(got, want_by_req, dtype, what):
    worst, over = 0.0, 0
    for (r, pos), row in got.items():
        want = want_by_req[r][pos]
        err = np.abs(row - want).max() / np.abs(want_by_req[r]).max()
        if dtype == "bfloat16" and TOLERANCE[dtype] < err <= max(BF16_WORST, 1.5 * ROUNDED[what.split("/")[0]][1]):
            over += 1
        else:
            assert err <= TOLERANCE[dtype], f"{what}: request {r} position {pos}: |diff| = {err:.3e} of max|logit| (allowed {TOLERANCE[dtype]:.0e})"
        worst = max(worst, err)
    assert len(got) == sum(len(v) for v in want_by_req.values())
    allowed = max(BF16_ROWS_OVER * len(got), 1.5 * ROUNDED[what.split("/")[0]][0]) if dtype == "bfloat16" else 0
    assert over <= allowed, f"{what}: {over} of {len(got)} rows are beyond {TOLERANCE[dtype]:.0e} of max|logit| (allowed {allowed:.0f})"
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tz.CONFIGS))
def test_layers_one_by_one(zdirs, name, dtype):
    """The residual stream after every layer against the plain model's, so that a wrong layer is named."""
    toks = _requests(name)["c"]
    want = P.PlainZabonex(zdirs[name]).hidden_states(toks)
    runner = _runner(zdirs, name, dtype, 64)
    from inference_bench_b200.engine.step import StepEntry
    runner.cache.admit("x")
    layers = []
    runner.step([StepEntry("x", toks, list(range(len(toks))))], trace=layers)
    assert len(layers) == len(want)
    for i, (g, w) in enumerate(zip(layers, want)):
        err = (g.cpu().double() - w).abs().amax(dim=1) / w.abs().max().item()      # per token
        where = f"{name}/{dtype}: the stream after {'the embedding' if i == 0 else f'layer {i - 1}'}"
        if dtype == "float32":
            assert err.max().item() < 2e-5, f"{where} differs by {err.max().item():.2e}"
        else:   # a token whose router choice fell the other way may differ more (see BF16_ROWS_OVER)
            rounded = P.PlainZabonex(zdirs[name]).hidden_states(toks, P.bf16)[i]
            ref = (rounded - w).abs().amax(dim=1) / w.abs().max().item()
            assert err.median().item() < max(1.5e-2, 3 * ref.median().item()) and (err > 4e-2).sum().item() <= 2 + 1.5 * (ref > 4e-2).sum().item() and \
                err.max().item() < max(BF16_WORST, 1.5 * ref.max().item()), f"{where} differs by {err.max().item():.2e} (median {err.median().item():.2e})"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tz.CONFIGS))
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
def test_cut_matches_plain(zdirs, plain_logits, name, dtype, cut):
    """Whole prompts; prompts then the last tokens one by one (a long tail for the longest request); portions down to two tokens;
    up to four live requests of unequal length in one batch with a pool that only holds what is live, so pages and slots are
    used again by later requests."""
    reqs = _requests(name)
    steps = {"whole": traces.whole, "tail": lambda r: traces.tail_one_by_one(r, tail=90), "portions": traces.portions, "mixed": traces.mixed}[cut](reqs)
    max_tokens = traces.max_live_tokens(steps)
    runner = _runner(zdirs, name, dtype, max_tokens, max_requests=4)
    got = traces.run_steps(runner, steps)
    worst = _compare(got, plain_logits[name], dtype, f"{name}/{dtype}/{cut}")
    runner.cache.check()
    assert runner.cache.used_pages() == [0] * len(runner.cache.groups)
    print(f"{name}/{dtype}/{cut}: worst {worst:.3e} of max|logit|, pool {max_tokens} tokens")


def test_a_request_alone_and_in_a_batch_give_the_same_float32_logits(zdirs):
    """The float32 path adds in one order whatever shares the step: a request beside three others of other lengths, on other pages
    and in another slot, gives the bits it gives alone."""
    from inference_bench_b200.engine.step import StepEntry
    name = "Q"
    reqs = _requests(name)
    runner = _runner(zdirs, name, "float32", 1024, max_requests=4)
    runner.cache.admit("alone")
    alone = runner.step([StepEntry("alone", reqs["d"], [len(reqs["d"]) - 1])]).cpu()
    runner.cache.release("alone")
    for r in ("b", "f", "d", "a"):
        runner.cache.admit(r)
    rows = runner.step([StepEntry(r, reqs[r], [len(reqs[r]) - 1]) for r in ("b", "f", "d", "a")]).cpu()
    assert torch.equal(rows[2], alone[0])


@pytest.mark.parametrize("name", list(tz.CONFIGS))
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_engine(zdirs, name, graphs):
    """`Engine.generate`: the scheduler cuts prompts into portions, batches them beside decoded tokens, and decode steps run as
    captured graphs or not; float32 tokens equal the plain model's."""
    from inference_bench_b200 import Engine
    vocab = tz.CONFIGS[name]["config"]["vocab"]
    plain = P.PlainZabonex(zdirs[name])
    prompts = [traces.prompt(70 + i, n, vocab) for i, n in enumerate((5, 21, 40))]
    want = [plain.greedy(p, 7) for p in prompts]
    eng = Engine(zdirs[name], dtype="float32", max_ctx=128, page_size=tz.CONFIGS[name]["page_size"], use_graphs=graphs, prefill_chunk=9, max_batched_tokens=16)
    got = eng.generate(prompts, max_tokens=7)
    assert [r.tokens for r in got] == want
    assert eng.cache.used_pages() == [0] * len(eng.cache.groups)
    eng.cache.check()
    one = eng.generate(prompts[1], max_tokens=7)
    assert one.tokens == want[1]


def test_generation_in_bfloat16_runs_and_long_decoding_stays_close(zdirs):
    from inference_bench_b200 import Engine
    name = "R"
    vocab = tz.CONFIGS[name]["config"]["vocab"]
    plain = P.PlainZabonex(zdirs[name])
    prompt = traces.prompt(5, 12, vocab)
    eng = Engine(zdirs[name], dtype="bfloat16", max_ctx=256, page_size=32)
    got = eng.generate(prompt, max_tokens=150).tokens
    assert len(got) == 150
    # teacher-forced on the engine's own tokens, the plain model ranks every chosen token near the top
    lg = plain.logits(prompt + got)
    for i, tok in enumerate(got):
        row = lg[len(prompt) + i - 1]
        assert row[tok] >= row.max() - 0.25, f"decoded token {i}: the plain model's logit for it is {row.max() - row[tok]:.3f} below its best"


# ------------------------------------------------------------------------------------------ the programs a user runs
def test_trace_replay_program_and_command_line(zdirs, tmp_path):
    """bin/trace_run as a subprocess fed JSON steps (a mixed trace, bfloat16), and `run`, `batch` and `spec` of the command line, on a
    model folder of this architecture: nothing in them names an architecture."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    name = "R"
    vocab = tz.CONFIGS[name]["config"]["vocab"]
    reqs = {r: traces.prompt(900 + i, n, vocab) for i, (r, n) in enumerate({"a": 70, "b": 9, "c": 33, "d": 64, "e": 2}.items())}
    steps = traces.mixed(reqs, seed=5)
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(zdirs[name]), "--dtype", "bfloat16", "--out", str(out),
                           "--max-tokens", str(traces.max_live_tokens(steps)), "--page-size", "32"],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    plain = P.PlainZabonex(zdirs[name])
    want = {r: plain.logits(t).numpy() for r, t in reqs.items()}
    at, over, n_rows = {r: 0 for r in reqs}, 0, 0
    for s in steps:
        rows = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab)
        k = 0
        for e in s["entries"]:
            for w in e["want"]:
                err = np.abs(rows[k] - want[e["id"]][at[e["id"]] + w]).max() / np.abs(want[e["id"]]).max()
                assert err <= BF16_WORST
                over += err > TOLERANCE["bfloat16"]
                k += 1
            at[e["id"]] += len(e["tokens"])
        assert k == rows.shape[0]
        n_rows += k
    assert over <= max(3, BF16_ROWS_OVER * n_rows)
    env = dict(os.environ, PYTHONPATH=root)
    p = subprocess.run([sys.executable, "-m", "inference_bench_b200", "run", "--model", str(zdirs[name]), "--prompt-len", "12", "--max-tokens", "5", "--json",
                        "--dtype", "float32", "--max-ctx", "64"], capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    r = json.loads(p.stdout)
    from inference_bench_b200.cli import _synthetic_prompt
    assert r["prompt_tokens"] == 12 and r["tokens"] == plain.greedy(_synthetic_prompt(12, vocab), 5)
    p = subprocess.run([sys.executable, "-m", "inference_bench_b200", "batch", "--model", str(zdirs[name]), "--sizes", "1,3", "--prompt-len", "20", "--max-tokens", "6",
                        "--json", "--max-ctx", "64"], capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [b["completion_tokens"] for b in json.loads(p.stdout)] == [6, 18]
    p = subprocess.run([sys.executable, "-m", "inference_bench_b200", "spec", "--model", str(zdirs[name])], capture_output=True, text=True, env=env)
    assert p.returncode == 0 and json.loads(p.stdout)["layers"][1]["mixer"]["kv_from"] == 0
