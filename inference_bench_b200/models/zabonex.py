"""Zabonex as a plan: latent-attention layers whose norms sit on the sublayers' outputs, dense or routed feed-forwards,
and layers that read an earlier layer's cached latent instead of making their own.

Tensor names: `embed`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.{q,dkv,dkv.norm,uk,uv,o}`, `l<i>.mlp.{gate,up,down}` or
`l<i>.mlp.{router, e<k>.{gate,up,down}, shared.{gate,up,down}}`, `final.norm`, `head`. They have no common root.
"""
from __future__ import annotations

from ..config.zabonex import ZabonexConfig
from ..parts.plan import LayerPlan, ModelPlan, PartSpec, ScheduleEntry
from ..registry import register_architecture

MAX_POSITIONS = 1 << 20   # the rotation has no table: positions are bounded by the cache alone


def zabonex_plan(c: ZabonexConfig) -> ModelPlan:
    layers, schedule = [], []
    for i, l in enumerate(c.layers):
        m, p = l.mixer, f"l{i}"
        rope = PartSpec("rope", {"rotary_dim": m.rot_dims, "theta": m.rot_base, "pairing": "interleaved"}) if m.rot_dims else PartSpec("none")
        mixer = PartSpec("latent_attention", {
            "prefix": f"{p}.mix", "hidden": c.width, "heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank,
            "scale": m.scale, "norm_eps": c.norm_eps, "position": rope, "own_kv": m.kv_from is None})
        if l.mlp is None:
            ff, ff_norm = PartSpec("none"), PartSpec("none")
        else:
            ff_norm = PartSpec("rmsnorm", {"name": f"{p}.norm2", "size": c.width, "eps": c.norm_eps, "unit_offset": True})
            if l.mlp.kind == "dense":
                ff = PartSpec("swiglu", {"prefix": f"{p}.mlp", "hidden": c.width, "intermediate": l.mlp.ff, "names": ("gate", "up", "down")})
            else:
                f = l.mlp
                ff = PartSpec("routed_experts", {
                    "prefix": f"{p}.mlp", "hidden": c.width, "expert_ff": f.ff, "experts": f.experts, "top": f.top, "route_scale": f.route_scale,
                    "groups": f.groups, "groups_keep": f.groups_keep, "shared_ff": f.shared_ff, "renorm": False})
        layers.append(LayerPlan(prefix=p, block="outnorm", mixer=mixer, feed_forward=ff,
                                mixer_norm=PartSpec("rmsnorm", {"name": f"{p}.norm1", "size": c.width, "eps": c.norm_eps, "unit_offset": True}),
                                feed_forward_norm=ff_norm, block_params=(("residual_mult", c.residual_mult),)))
        schedule.append(ScheduleEntry(i, cache_of=m.kv_from))   # one execution per layer, so a layer's number is its entry's
    return ModelPlan(
        architecture="Zabonex", vocab_size=c.vocab, hidden_size=c.width, max_positions=MAX_POSITIONS,
        embedding=PartSpec("table", {"name": "embed", "vocab": c.vocab, "hidden": c.width}),
        layers=tuple(layers), schedule=tuple(schedule),
        final_norm=PartSpec("rmsnorm", {"name": "final.norm", "size": c.width, "eps": c.norm_eps, "unit_offset": True}),
        head=PartSpec("linear", {"name": "head", "vocab": c.vocab, "hidden": c.width}),
        root="",
    )


register_architecture(["Zabonex", "zabonex"], ZabonexConfig.from_dict, zabonex_plan,
                      traits={"attention": "latent", "qk_norm": False, "norm": "rmsnorm", "norm_unit_offset": True, "rope_style": "interleaved", "activation": "swiglu"})
