"""Tiny Zabonex configurations for the tests, with weights the tests make themselves. They differ in every size and
constant: width (a multiple of 8 or not), heads (fewer than, more than and no multiple of the eight heads an attention CTA
takes), per-head sizes, latent size (a multiple of 32 or not), rotated part (all of it turned, or only its first entries), the
order of layers with a latent of their own and layers that read another's (the layer before, or one further back), dense,
routed (with and without groups, one or several experts a token, with and without a shared expert) and absent feed-forwards,
residual multiplier, router scale, norm epsilon, rotation base."""
from __future__ import annotations

import json
from pathlib import Path

import torch


def _mixer(heads, dim, rot_dim, vdim, rank, base, dims=None, kv_from=None, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale if scale is not None else (dim + rot_dim) ** -0.5,
         "rot": {"base": base, "dims": rot_dim if dims is None else dims}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _moe(ff, experts, top, scale, groups=None, shared=None):
    r = {"experts": experts, "top": top, "scale": scale}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    f = {"kind": "moe", "expert": {"ff": ff}, "router": r}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def _layer(mixer, mlp):
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


_P = dict(heads=3, dim=24, rot_dim=8, vdim=20, rank=40, base=1000.0)
_Q = dict(heads=11, dim=16, rot_dim=12, vdim=10, rank=72, base=50000.0, dims=6)
_R = dict(heads=16, dim=32, rot_dim=16, vdim=48, rank=128, base=8000.0)

CONFIGS = {
    # three heads; layer 1 reads layer 0's latent, layer 3 reads it too (two layers back); one expert a token without groups or shared expert
    "P": dict(seed=11, page_size=16, config={
        "architecture": "Zabonex", "vocab": 300, "width": 80, "norm": {"eps": 1e-6}, "residual_mult": 1.0,
        "layers": [_layer(_mixer(**_P), {"kind": "dense", "ff": 112}),
                   _layer(_mixer(**_P, kv_from=0), _moe(40, 5, 1, 1.0)),
                   _layer(_mixer(**_P, scale=0.3), _moe(24, 6, 2, 0.5, groups=(3, 1), shared=56)),
                   _layer(_mixer(**_P, kv_from=0), {"kind": "dense", "ff": 64})]}),
    # eleven heads (two attention CTAs a token, the second partly filled), a width that is no multiple of 8, a latent that is no
    # multiple of 32, only half of the rotated part turned, a layer without a feed-forward, small pages
    "Q": dict(seed=12, page_size=8, config={
        "architecture": "Zabonex", "vocab": 257, "width": 132, "norm": {"eps": 1e-5}, "residual_mult": 0.35,
        "layers": [_layer(_mixer(**_Q), _moe(36, 16, 4, 2.5, groups=(4, 2), shared=20)),
                   _layer(_mixer(**_Q), None),
                   _layer(_mixer(**_Q, kv_from=1), {"kind": "dense", "ff": 100})]}),
    # sixteen heads, sizes that are multiples of 16 and 32, larger pages
    "R": dict(seed=13, page_size=32, config={
        "architecture": "Zabonex", "vocab": 512, "width": 256, "norm": {"eps": 1e-5}, "residual_mult": 0.6,
        "layers": [_layer(_mixer(**_R), _moe(64, 8, 2, 1.5, groups=(4, 2), shared=128)),
                   _layer(_mixer(**_R, kv_from=0), {"kind": "dense", "ff": 320})]}),
}


def tensors(config: dict, seed: int, sharp: float = 1.0) -> dict[str, torch.Tensor]:
    """Random bfloat16 tensors for a configuration: matrices N(0, 1/sqrt(fan-in)), so that activations stay of order one through
    every product and attention and routing are neither flat nor one-hot; norm weights around zero (layer and final norms) or
    around one (the latent's). `sharp` scales the query matrices: larger values make attention peak."""
    g = torch.Generator().manual_seed(seed)
    W, out = config["width"], {}

    def mat(name, n, k, gain=1.0):
        out[name] = (torch.randn((n, k), generator=g) * gain / k ** 0.5).to(torch.bfloat16)

    def vec(name, n, centre):
        out[name] = (centre + (torch.rand((n,), generator=g) * 0.6 - 0.3)).to(torch.bfloat16)

    out["embed"] = torch.randn((config["vocab"], W), generator=g).to(torch.bfloat16)
    for i, l in enumerate(config["layers"]):
        m, p = l["mixer"], f"l{i}"
        H = m["heads"]
        vec(f"{p}.norm1", W, 0.0)
        mat(f"{p}.mix.q", H * (m["dim"] + m["rot_dim"]), W, 2.0 * sharp)
        if m.get("kv_from") is None:
            mat(f"{p}.mix.dkv", m["kv_rank"] + m["rot_dim"], W, 2.0)
            vec(f"{p}.mix.dkv.norm", m["kv_rank"], 1.0)
        mat(f"{p}.mix.uk", H * m["dim"], m["kv_rank"], 2.0)
        mat(f"{p}.mix.uv", H * m["vdim"], m["kv_rank"])
        mat(f"{p}.mix.o", W, H * m["vdim"])
        f = l.get("mlp")
        if f is None:
            continue
        vec(f"{p}.norm2", W, 0.0)
        if f["kind"] == "dense":
            mat(f"{p}.mlp.gate", f["ff"], W), mat(f"{p}.mlp.up", f["ff"], W), mat(f"{p}.mlp.down", W, f["ff"])
            continue
        mat(f"{p}.mlp.router", f["router"]["experts"], W, 2.0)
        for k in range(f["router"]["experts"]):
            mat(f"{p}.mlp.e{k}.gate", f["expert"]["ff"], W), mat(f"{p}.mlp.e{k}.up", f["expert"]["ff"], W), mat(f"{p}.mlp.e{k}.down", W, f["expert"]["ff"])
        if f.get("shared"):
            s = f["shared"]["ff"]
            mat(f"{p}.mlp.shared.gate", s, W), mat(f"{p}.mlp.shared.up", s, W), mat(f"{p}.mlp.shared.down", W, s)
    vec("final.norm", W, 0.0)
    mat("head", config["vocab"], W)
    return out


def write_model(name: str, out_dir, sharp: float = 1.0) -> Path:
    from inference_bench_b200.weights.safetensors_io import write_safetensors
    c = CONFIGS[name]
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    (out / "config.json").write_text(json.dumps(c["config"], indent=1))
    write_safetensors(out / "model.safetensors", tensors(c["config"], c["seed"], sharp), {"format": "pt"})
    return out
