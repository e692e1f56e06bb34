"""Busadra as a plan: pre-norm layers with layer norms, an input convolution in front of every sublayer, per-channel scales on the
sublayers' contributions and a depth-weighted average after every layer; mixers are windowed attention (biases, partly turned heads
with rescaled frequencies, capped scores, a softmax with one added to its denominator) or a gated linear recurrence; feed-forwards are
experts chosen by sigmoid scores whose weight scales the expert's input.

Tensor names: `embed`, `l<i>.{norm1,norm2,ls1,ls2,canon1,canon2,dwa}`, `l<i>.mix.{q,k,v,o}` with `.b` biases or
`l<i>.mix.{q,f,f.b,lower,v,norm,o}`, `l<i>.mlp.{router, e<k>.{gate,up,down}}`, `final.norm`, `head`. They have no common root.
"""
from __future__ import annotations

from ..config.busadra import BusadraConfig
from ..parts.plan import LayerPlan, ModelPlan, PartSpec, ScheduleEntry
from ..registry import register_architecture

MAX_POSITIONS = 1 << 20   # the rotation has no table: positions are bounded by the cache alone


def busadra_plan(c: BusadraConfig) -> ModelPlan:
    layers = []
    for i, l in enumerate(c.layers):
        m, p = l.mixer, f"l{i}"
        if l.type == "attention":
            s = m.rot_scaling
            rope = PartSpec("rope", {"rotary_dim": m.rot_dims, "theta": m.rot_base,
                                     "scaling": None if s is None else (s.factor, s.low, s.high, s.original)}) if m.rot_dims else PartSpec("none")
            mixer = PartSpec("attention", {
                "prefix": f"{p}.mix", "hidden": c.width, "heads": m.heads, "kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim, "qk_norm": False,
                "norm_eps": c.norm_eps, "position": rope, "window": m.window, "scale": m.scale, "bias": True, "softcap": m.softcap, "sink": True,
                "names": ("q", "k", "v", "o", "q.norm", "k.norm", "{}.b")})
        else:
            mixer = PartSpec("hgrn2", {"prefix": f"{p}.mix", "hidden": c.width, "heads": m.heads, "dim": m.dim, "vdim": m.vdim, "norm_eps": c.norm_eps})
        if l.mlp is None:
            ff, ff_norm = PartSpec("none"), PartSpec("none")
        else:
            ff_norm = PartSpec("layernorm", {"name": f"{p}.norm2", "size": c.width, "eps": c.norm_eps})
            ff = PartSpec("routed_experts", {"prefix": f"{p}.mlp", "hidden": c.width, "expert_ff": l.mlp.ff, "experts": l.mlp.experts, "top": l.mlp.top,
                                             "score": "sigmoid", "weight_on": "input"})
        layers.append(LayerPlan(prefix=p, block="prenorm_canon", mixer=mixer, feed_forward=ff,
                                mixer_norm=PartSpec("layernorm", {"name": f"{p}.norm1", "size": c.width, "eps": c.norm_eps}), feed_forward_norm=ff_norm,
                                block_params=(("prefix", p), ("hidden", c.width), ("taps", c.canon_taps), ("index", i), ("depth", len(c.layers)))))
    return ModelPlan(
        architecture="Busadra", vocab_size=c.vocab, hidden_size=c.width, max_positions=MAX_POSITIONS,
        embedding=PartSpec("table", {"name": "embed", "vocab": c.vocab, "hidden": c.width}),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=PartSpec("layernorm", {"name": "final.norm", "size": c.width, "eps": c.norm_eps}),
        head=PartSpec("linear", {"name": "head", "vocab": c.vocab, "hidden": c.width, "scale": c.logit_scale}),
        root="",
    )


register_architecture(["Busadra", "busadra"], BusadraConfig.from_dict, busadra_plan,
                      traits={"attention": "gqa", "qk_norm": False, "norm": "layernorm", "norm_unit_offset": False, "rope_style": "neox", "activation": "swiglu"})
