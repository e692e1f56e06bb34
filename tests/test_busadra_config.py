"""Busadra without a device: its configuration, its plan, its tensors, what it asks of the cache manager, and the plain model's own pieces."""
from __future__ import annotations

import copy
import math

import pytest
import torch

import plain_busadra as P
import tiny_busadra as tb
from inference_bench_b200.config import ConfigError
from inference_bench_b200.engine.model import plan_from_config
from inference_bench_b200.parts.base import FixedState, PagedKV, Several
from inference_bench_b200.parts.decoder import Decoder


@pytest.mark.parametrize("name", list(tb.CONFIGS))
def test_configuration_plan_and_tensors(name):
    raw = tb.CONFIGS[name]["config"]
    cfg, plan = plan_from_config(raw)
    assert plan.architecture == "Busadra" and len(plan.layers) == len(raw["layers"]) and plan.root == ""
    again = cfg.to_dict()
    assert again["layers"] == raw["layers"] and again["canon"] == raw["canon"] and again["logit_scale"] == raw.get("logit_scale", 1.0)
    d = Decoder(plan)
    made = tb.tensors(raw, 1)
    specs = {s.name: tuple(s.shape) for s in d.weight_specs()}
    assert specs == {n: tuple(t.shape) for n, t in made.items()}
    taps, W = raw["canon"]["taps"], raw["width"]
    for need, l in zip(d.cache_needs(), raw["layers"]):
        assert isinstance(need, Several) and need.needs[1] == FixedState((2, max(taps - 1, 1), W), torch.float32)
        m = l["mixer"]
        if l["type"] == "attention":
            assert need.needs[0] == PagedKV(m["kv_heads"], max(m["dim"], m["vdim"]), m["mask"]["size"])
        else:
            assert need.needs[0] == FixedState((m["heads"], m["dim"], m["vdim"]), torch.float32)


def test_cache_manager_takes_several_needs_of_one_layer():
    from inference_bench_b200.cache.manager import CacheManager
    d = Decoder(plan_from_config(tb.CONFIGS["A"]["config"])[1])
    cache = CacheManager(d.cache_needs(), 16, 8, 2, 64, sources=d.cache_sources())
    assert len(cache.groups) == 2 and [g.window for g in cache.groups] == [24, 9]       # two attention layers, two windows
    assert set(cache.place) == {(1, 0), (2, 0)} and set(cache.states) == {(0, 0), (0, 1), (1, 1), (2, 1), (3, 0), (3, 1)}
    views = cache.views([None, None])
    assert all(isinstance(v, tuple) and len(v) == 2 for v in views)
    cache.admit("a")
    cache.extend("a", 40)
    cache.commit("a", 40)
    assert cache.used_pages() == [2, 1]      # the windows let the pages that passed go
    cache.release("a")
    cache.check()


@pytest.mark.parametrize("change,why", [
    (lambda c: c["layers"][0].update(type="conv"), "not supported"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=34), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].update(softcap=0.0), "softcap"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top 9"),
    (lambda c: c["canon"].update(taps=0), "taps"),
    (lambda c: c.pop("canon"), "canon"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "not supported"),
])
def test_refusals(change, why):
    raw = copy.deepcopy(tb.CONFIGS["A"]["config"])
    change(raw)
    with pytest.raises(ConfigError, match=why):
        plan_from_config(raw)


def test_rescaled_frequencies_fall_in_three_bands():
    """With a short original length the bands all occur: the fastest entries stay, the slowest are divided by the factor, the ones
    between lie between; the engine's table agrees with the plain model's."""
    from inference_bench_b200.parts.standard import RotaryEmbedding
    rot = {"base": 1000.0, "dims": 16, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}
    plain = torch.tensor([1000.0 ** (-2.0 * i / 16) for i in range(8)], dtype=torch.float64)
    got = P.rotary_frequencies(rot)
    ratio = (got / plain).tolist()
    assert ratio[0] == 1.0 and ratio[-1] == pytest.approx(1 / 8) and any(1 / 8 + 1e-6 < r < 1 - 1e-6 for r in ratio)
    assert sorted(ratio, reverse=True) == ratio

    class _Rt:
        @staticmethod
        def upload(t):
            return t
    r = RotaryEmbedding(16, 1000.0, scaling=(8.0, 1.0, 4.0, 64))
    r.bind({}, _Rt)
    assert torch.allclose(r.inv_freq.double(), got, rtol=1e-6)
    r = RotaryEmbedding(16, 1000.0)
    r.bind({}, _Rt)
    assert torch.allclose(r.inv_freq.double(), plain, rtol=1e-6)


def test_plain_pieces_agree_with_their_definitions():
    g = torch.Generator().manual_seed(3)
    x = torch.randn((5, 12), generator=g, dtype=torch.float64)
    w = torch.rand((12,), generator=g, dtype=torch.float64)
    assert torch.allclose(P.layer_norm(x, w, 1e-5), torch.nn.functional.layer_norm(x, (12,), w, None, 1e-5))
    taps = torch.randn((12, 3), generator=g, dtype=torch.float64)
    y = P.causal_conv(x, taps)
    assert torch.allclose(y[0], taps[:, 2] * x[0]) and torch.allclose(y[3], taps[:, 0] * x[1] + taps[:, 1] * x[2] + taps[:, 2] * x[3])
    # the sink: a lone key of score s gets weight e^s / (1 + e^s)
    q, k, v = torch.full((1, 1, 2), 1.0), torch.full((1, 1, 2), 0.5), torch.tensor([[[3.0, -1.0]]])
    out = P.attention_core(q, k, v, scale=2.0, cap=None, window=4)
    assert torch.allclose(out[0, 0], torch.tensor([3.0, -1.0], dtype=torch.float64) * (math.e ** 2 / (1 + math.e ** 2)))
    # the recurrence: with f = 0 the state is the last outer product, with f = 1 it never changes
    o, S = P.recurrence_core(torch.ones((2, 1, 2)), torch.zeros((2, 1, 2)), torch.tensor([[[1.0, 2.0]], [[3.0, 4.0]]]))
    assert torch.allclose(S[0], torch.tensor([[3.0, 4.0], [3.0, 4.0]], dtype=torch.float64)) and torch.allclose(o[1, 0], torch.tensor([6.0, 8.0], dtype=torch.float64))
    o, S = P.recurrence_core(torch.ones((2, 1, 2)), torch.ones((2, 1, 2)), torch.ones((2, 1, 2)))
    assert float(S.abs().max()) == 0.0
