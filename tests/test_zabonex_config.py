"""Zabonex without a device: reading config.json, the plan it becomes, the tensors it declares, weights written and read back,
the cache's bookkeeping for rows that several layers read, and the plain implementation's own pieces."""
from __future__ import annotations

import copy
import json

import pytest
import torch

import plain_zabonex as P
import tiny_zabonex as tz
from inference_bench_b200.config import ConfigError
from inference_bench_b200.config.zabonex import ZabonexConfig
from inference_bench_b200.engine.model import plan_from_config
from inference_bench_b200.parts.base import PagedRows
from inference_bench_b200.parts.decoder import Decoder


@pytest.mark.parametrize("name", list(tz.CONFIGS))
def test_config_reads_every_size_and_reads_back(name):
    raw = tz.CONFIGS[name]["config"]
    cfg = ZabonexConfig.from_dict(raw)
    assert cfg.width == raw["width"] and cfg.vocab == raw["vocab"] and cfg.residual_mult == raw["residual_mult"] and cfg.norm_eps == raw["norm"]["eps"]
    for l, r in zip(cfg.layers, raw["layers"]):
        m = r["mixer"]
        assert (l.mixer.heads, l.mixer.dim, l.mixer.rot_dim, l.mixer.vdim, l.mixer.kv_rank, l.mixer.scale) == (m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["scale"])
        assert (l.mixer.rot_base, l.mixer.rot_dims, l.mixer.kv_from) == (m["rot"]["base"], m["rot"]["dims"], m.get("kv_from"))
        assert (l.mlp is None) == (r["mlp"] is None)
    assert ZabonexConfig.from_dict(cfg.to_dict()) == cfg
    assert ZabonexConfig.from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg


def test_config_refuses_what_the_design_does_not_have():
    raw = tz.CONFIGS["P"]["config"]

    def broken(change):
        c = copy.deepcopy(raw)
        change(c)
        return c

    cases = [
        (lambda c: c["layers"][0].update(type="window_attention"), "not supported"),
        (lambda c: c["layers"][1]["mixer"].update(kv_from=1), "earlier layer"),
        (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "keeps no latent"),
        (lambda c: c["layers"][1]["mixer"].update(kv_rank=48), "differ"),
        (lambda c: c["layers"][2]["mlp"]["router"]["groups"].update(count=4), "equal groups"),
        (lambda c: c["layers"][2]["mlp"]["router"].update(top=3), "exceeds"),
        (lambda c: c["layers"][0]["mlp"].update(kind="conv"), "not supported"),
        (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "rot.dims"),
        (lambda c: c.pop("width"), "width"),
        (lambda c: c["layers"][0]["mixer"].pop("vdim"), "vdim"),
    ]
    for change, word in cases:
        with pytest.raises(ConfigError, match=word):
            ZabonexConfig.from_dict(broken(change))


def test_the_architecture_is_found_by_its_name_in_the_singular_key():
    from inference_bench_b200.registry import resolve
    assert resolve({"architecture": "Zabonex"}).name == "Zabonex"
    assert resolve({"architectures": ["Zabonex"]}).name == "Zabonex"
    with pytest.raises(ConfigError):
        resolve({"architecture": "Nobody"})


@pytest.mark.parametrize("name", list(tz.CONFIGS))
def test_plan_declares_the_tensors_and_the_shared_caches(name):
    raw = tz.CONFIGS[name]["config"]
    _, plan = plan_from_config(raw)
    d = Decoder(plan)
    want = {k: tuple(v.shape) for k, v in tz.tensors(raw, 0).items()}
    assert {s.name: tuple(s.shape) for s in d.weight_specs()} == want
    needs, sources = d.cache_needs(), d.cache_sources()
    for i, l in enumerate(raw["layers"]):
        m = l["mixer"]
        if m.get("kv_from") is None:
            assert needs[i] == PagedRows(m["kv_rank"] + m["rot_dim"]) and sources[i] == i
        else:
            assert needs[i] is None and sources[i] == m["kv_from"]


def test_weights_written_and_loaded_by_name(tmp_path):
    from inference_bench_b200.weights.loader import WeightError, load_weights
    from inference_bench_b200.weights.safetensors_io import write_safetensors
    folder = tz.write_model("Q", tmp_path / "q")
    _, plan = plan_from_config(json.loads((folder / "config.json").read_text()))
    d = Decoder(plan)
    got = load_weights(folder, d.weight_specs(), root=plan.root)
    want = tz.tensors(tz.CONFIGS["Q"]["config"], tz.CONFIGS["Q"]["seed"])
    assert set(got) == set(want) and all(torch.equal(got[k], want[k]) for k in want)
    short = dict(want)
    short.pop("l2.mix.uk")
    short["l0.mix.dkv.norm"] = short["l0.mix.dkv.norm"][:-1]
    write_safetensors(tmp_path / "q" / "model.safetensors", short, {})
    with pytest.raises(WeightError) as e:
        load_weights(folder, d.weight_specs(), root=plan.root)
    assert e.value.missing == ["l2.mix.uk"] and [w[0] for w in e.value.wrong_shape] == ["l0.mix.dkv.norm"]


def test_random_weights_for_the_architecture(tmp_path):
    from inference_bench_b200.weights.random_init import write_random_model
    folder = write_random_model(tz.CONFIGS["P"]["config"], 3, tmp_path / "p")
    m = P.PlainZabonex(folder)
    assert abs(float(m.weights["l0.norm1"].float().mean())) < 0.1 and abs(float(m.weights["l0.mix.dkv.norm"].float().mean()) - 1.0) < 0.1
    assert torch.isfinite(m.logits([1, 2, 3])).all()


def test_cache_rows_are_one_group_for_all_layers_that_keep_them():
    from inference_bench_b200.cache.manager import CacheManager
    _, plan = plan_from_config(tz.CONFIGS["P"]["config"])
    d = Decoder(plan)
    cache = CacheManager(d.cache_needs(), 16, 6, 2, 64, sources=d.cache_sources())
    assert len(cache.groups) == 1 and cache.groups[0].entries == [0, 2] and cache.place == {0: (0, 0), 2: (0, 1)}
    cache.admit("a")
    cache.extend("a", 40)
    cache.commit("a", 40)
    assert cache.used_pages() == [3]
    cache.admit("b")
    with pytest.raises(Exception):
        cache.extend("b", 64)          # four pages wanted, three left
    cache.release("a")
    cache.extend("b", 64)
    cache.commit("b", 64)
    assert cache.used_pages() == [4]
    cache.release("b")
    cache.check()
    assert cache.used_pages() == [0]


# ------------------------------------------------------------------------------------------ the plain implementation's own pieces
def test_plain_rotation_turns_pairs_and_keeps_the_rest():
    v = torch.arange(12, dtype=torch.float64).reshape(1, 2, 6) + 1
    out = P.rotate_pairs(v, torch.tensor([0, 3]), 100.0, 4)
    assert torch.equal(out[0, 0], v[0, 0])                      # position 0: nothing turns
    assert torch.equal(out[0, 1, 4:], v[0, 1, 4:])              # beyond `dims`: untouched
    a, b = v[0, 1, 0], v[0, 1, 1]
    assert torch.allclose(out[0, 1, 0], a * torch.cos(torch.tensor(3.0, dtype=torch.float64)) - b * torch.sin(torch.tensor(3.0, dtype=torch.float64)))
    ang = torch.tensor(3.0 * 100.0 ** -0.5, dtype=torch.float64)
    assert torch.allclose(out[0, 1, 3], v[0, 1, 3] * torch.cos(ang) + v[0, 1, 2] * torch.sin(ang))
    assert torch.allclose(out.norm(), v.norm())


def test_plain_router_keeps_groups_before_experts():
    logits = torch.tensor([[5.0, 4.9, 0.0, 0.0, 4.0, 0.0]], dtype=torch.float64)
    eye = torch.eye(6, dtype=torch.float64)
    idx, wt = P.route(logits, eye, {"experts": 6, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 1}})
    assert sorted(idx[0].tolist()) == [0, 1]
    s = torch.softmax(logits, dim=-1)[0]
    assert torch.allclose(wt[0].sort().values, (2.0 * s[[1, 0]]))
    idx, _ = P.route(logits, eye, {"experts": 6, "top": 2, "scale": 1.0, "groups": {"count": 3, "keep": 2}})
    assert sorted(idx[0].tolist()) == [0, 1]
    idx, _ = P.route(logits, eye, {"experts": 6, "top": 3, "scale": 1.0, "groups": {"count": 3, "keep": 2}})
    assert sorted(idx[0].tolist()) == [0, 1, 4]
    idx, _ = P.route(logits, eye, {"experts": 6, "top": 3, "scale": 1.0})
    assert sorted(idx[0].tolist()) == [0, 1, 4]


def test_plain_attention_in_the_latent_equals_attention_on_keys_and_values():
    """The plain model builds every head's keys and values; the sum it computes is the one over the cached rows with the two
    per-head maps moved to the query and the output."""
    cfg = tz.CONFIGS["P"]["config"]
    m = cfg["layers"][0]["mixer"]
    w = {k: v.double() for k, v in tz.tensors(cfg, 5).items()}
    n = 9
    h = torch.randn((n, cfg["width"]), dtype=torch.float64, generator=torch.Generator().manual_seed(1))
    pos = torch.arange(n)
    c, kr = P.latent_kv(h, w, "l0.mix", m, 1e-6, pos)
    want = P.latent_attention(h, w, "l0.mix", m, c, kr, pos)
    H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ w["l0.mix.q"].T).view(n, H, dn + dr)
    qr = P.rotate_pairs(q[..., dn:].transpose(0, 1), pos, m["rot"]["base"], m["rot"]["dims"]).transpose(0, 1)
    uk, uv = w["l0.mix.uk"].view(H, dn, r), w["l0.mix.uv"].view(H, dv, r)
    rows = torch.cat([c, kr], dim=1)
    out = torch.zeros((n, H, dv), dtype=torch.float64)
    for t in range(n):
        for a in range(H):
            qa = torch.cat([uk[a].T @ q[t, a, :dn], qr[t, a]])
            p = torch.softmax((rows[:t + 1] @ qa) * m["scale"], dim=0)
            out[t, a] = uv[a] @ (p @ c[:t + 1])
    assert torch.allclose(out.reshape(n, H * dv) @ w["l0.mix.o"].T, want, atol=1e-10)
