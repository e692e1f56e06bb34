"""Tiny Busadra configurations for the tests, with weights the tests make themselves. They differ in every size and constant: width
(a multiple of 8 or not), the order of attention and recurrence layers, query and key/value head counts (equal, grouped by two and by
four), key and value sizes (equal or not), how much of a head is turned and whether its frequencies are rescaled (with an original
length so short that all three bands occur), windows shorter and longer than the prompts, caps, scales, the convolution's length (one
tap: no state; three; five), experts a token (one, two, four), layers without a feed-forward (after attention and after a
recurrence), logit scale, norm epsilon, page size."""
from __future__ import annotations

import json
from pathlib import Path

import torch


def _att(heads, kv_heads, dim, vdim, window, dims, base, scale, softcap, scaling=None):
    rot = {"base": base, "dims": dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window}, "rot": rot, "scale": scale, "softcap": softcap}


def _rec(heads, dim, vdim):
    return {"heads": heads, "dim": dim, "vdim": vdim}


def _moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


CONFIGS = {
    # recurrence first; grouped attention whose values are smaller than its keys and whose heads are half turned, with rescaled frequencies;
    # layers without a feed-forward after attention and after a recurrence; two experts a token
    "A": dict(seed=21, page_size=16, config={
        "architecture": "Busadra", "vocab": 300, "width": 80, "norm": {"eps": 1e-5}, "canon": {"taps": 3}, "logit_scale": 1.7,
        "layers": [_layer("hgrn2", _rec(3, 16, 24), _moe(24, 5, 2)),
                   _layer("attention", _att(4, 2, 32, 16, 24, 16, 1000.0, 0.3, 8.0, scaling=(8.0, 1.0, 4.0, 64)), _moe(40, 6, 2)),
                   _layer("attention", _att(4, 2, 32, 16, 9, 32, 300.0, 0.2, 30.0), None),
                   _layer("hgrn2", _rec(2, 40, 8), None)]}),
    # a width that is no multiple of 8; one tap (no convolution state); values larger than keys; a window longer than every prompt; no logit
    # scale; one expert a token; a recurrence with one head; small pages
    "B": dict(seed=22, page_size=8, config={
        "architecture": "Busadra", "vocab": 257, "width": 132, "norm": {"eps": 1e-6}, "canon": {"taps": 1},
        "layers": [_layer("attention", _att(6, 6, 24, 40, 1000, 8, 50000.0, 0.25, 15.0), _moe(36, 7, 1)),
                   _layer("hgrn2", _rec(1, 48, 20), _moe(20, 4, 1)),
                   _layer("attention", _att(3, 1, 16, 16, 13, 0, 10.0, 0.5, 5.0), _moe(36, 7, 1))]}),
    # heads of 64 and 128 with keys as large as values (the sizes the tensor-core attention kernels take), groups of four, five taps, four
    # experts a token, larger pages
    "C": dict(seed=23, page_size=32, config={
        "architecture": "Busadra", "vocab": 512, "width": 256, "norm": {"eps": 1e-5}, "canon": {"taps": 5}, "logit_scale": 0.25,
        "layers": [_layer("attention", _att(8, 2, 64, 64, 48, 64, 10000.0, 0.125, 50.0, scaling=(4.0, 1.0, 4.0, 256)), _moe(64, 16, 4)),
                   _layer("hgrn2", _rec(4, 64, 64), _moe(64, 8, 2)),
                   _layer("attention", _att(4, 1, 128, 128, 17, 32, 500.0, 0.09, 10.0), _moe(128, 4, 1))]}),
}


def tensors(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """Random bfloat16 tensors: matrices N(0, gain / sqrt(fan-in)) so that activations stay of order one, norm weights and per-channel
    scales around one, convolution taps N(0, 0.3), average weights around 1 / n, gate floors in (0, 0.9), biases N(0, 0.3)."""
    g = torch.Generator().manual_seed(seed)
    W, out = config["width"], {}
    taps = config["canon"]["taps"]

    def mat(name, n, k, gain=1.0):
        out[name] = (torch.randn((n, k), generator=g) * gain / k ** 0.5).to(torch.bfloat16)

    def vec(name, n, centre, spread=0.3):
        out[name] = (centre + (torch.rand((n,), generator=g) * 2 - 1) * spread).to(torch.bfloat16)

    def noise(name, shape, std):
        out[name] = (torch.randn(shape, generator=g) * std).to(torch.bfloat16)

    out["embed"] = torch.randn((config["vocab"], W), generator=g).to(torch.bfloat16)
    for i, l in enumerate(config["layers"]):
        m, p = l["mixer"], f"l{i}"
        H = m["heads"]
        vec(f"{p}.norm1", W, 1.0), vec(f"{p}.ls1", W, 0.8), noise(f"{p}.canon1", (W, taps), 0.3)
        out[f"{p}.dwa"] = ((0.7 + 0.6 * torch.rand((i + 2,), generator=g)) / (i + 2)).to(torch.bfloat16)
        if l["type"] == "attention":
            G = m["kv_heads"]
            mat(f"{p}.mix.q", H * m["dim"], W, 2.0), mat(f"{p}.mix.k", G * m["dim"], W, 2.0), mat(f"{p}.mix.v", G * m["vdim"], W), mat(f"{p}.mix.o", W, H * m["vdim"])
            noise(f"{p}.mix.q.b", (H * m["dim"],), 0.3), noise(f"{p}.mix.k.b", (G * m["dim"],), 0.3), noise(f"{p}.mix.v.b", (G * m["vdim"],), 0.3)
            noise(f"{p}.mix.o.b", (W,), 0.3)
        else:
            mat(f"{p}.mix.q", H * m["dim"], W), mat(f"{p}.mix.f", H * m["dim"], W, 2.0), mat(f"{p}.mix.v", H * m["vdim"], W), mat(f"{p}.mix.o", W, H * m["vdim"])
            noise(f"{p}.mix.f.b", (H * m["dim"],), 1.0)
            out[f"{p}.mix.lower"] = (torch.rand((H * m["dim"],), generator=g) * 0.9).to(torch.bfloat16)
            vec(f"{p}.mix.norm", m["vdim"], 1.0)
        f = l.get("mlp")
        if f is None:
            continue
        vec(f"{p}.norm2", W, 1.0), vec(f"{p}.ls2", W, 0.8), noise(f"{p}.canon2", (W, taps), 0.3)
        mat(f"{p}.mlp.router", f["router"]["experts"], W, 2.0)
        for k in range(f["router"]["experts"]):
            mat(f"{p}.mlp.e{k}.gate", f["expert"]["ff"], W, 2.0), mat(f"{p}.mlp.e{k}.up", f["expert"]["ff"], W, 2.0), mat(f"{p}.mlp.e{k}.down", W, f["expert"]["ff"])
    vec("final.norm", W, 1.0)
    mat("head", config["vocab"], W)
    return out


def write_model(name: str, out_dir) -> Path:
    from inference_bench_b200.weights.safetensors_io import write_safetensors
    c = CONFIGS[name]
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    (out / "config.json").write_text(json.dumps(c["config"], indent=1))
    write_safetensors(out / "model.safetensors", tensors(c["config"], c["seed"]), {"format": "pt"})
    return out
