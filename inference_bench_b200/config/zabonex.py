"""Typed configuration of the Zabonex decoder, read from its own config.json keys.

A Zabonex model is a list of layers, each with a latent-attention mixer and a feed-forward that is dense, a mixture
of experts, or absent. config.json gives every size and every constant; nothing here fixes one.

    architecture   "Zabonex"
    vocab, width   vocabulary size and width of the residual stream
    norm.eps       epsilon of every RMS norm
    residual_mult  factor on every normed sublayer output before it is added to the stream
    layers[i]      type ("latent_attention"), mixer {heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims}, kv_from?},
                   mlp null | {kind "dense", ff} | {kind "moe", expert {ff}, router {experts, top, scale, groups {count, keep}}, shared {ff}?}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional

from . import ConfigError

MIXER_TYPES = ("latent_attention",)
MLP_KINDS = ("dense", "moe")


def _need(d: Mapping[str, Any], key: str, where: str):
    if not isinstance(d, Mapping) or d.get(key) is None:
        raise ConfigError(f"config.json has no {where}.{key}")
    return d[key]


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int            # unrotated query/key values per head
    rot_dim: int        # rotated query/key values per head (the key's are shared by all heads)
    vdim: int           # value size per head
    kv_rank: int        # size of the cached latent
    scale: float        # factor on the scores
    rot_base: float
    rot_dims: int       # how many of the rot_dim values are turned
    kv_from: Optional[int] = None   # the layer whose cached latent and key part this layer reads instead of making its own

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "LatentMixerConfig":
        rot = _need(m, "rot", where)
        c = cls(heads=int(_need(m, "heads", where)), dim=int(_need(m, "dim", where)), rot_dim=int(_need(m, "rot_dim", where)),
                vdim=int(_need(m, "vdim", where)), kv_rank=int(_need(m, "kv_rank", where)), scale=float(_need(m, "scale", where)),
                rot_base=float(_need(rot, "base", where + ".rot")), rot_dims=int(_need(rot, "dims", where + ".rot")),
                kv_from=None if m.get("kv_from") is None else int(m["kv_from"]))
        for name in ("heads", "dim", "vdim", "kv_rank"):
            if getattr(c, name) <= 0:
                raise ConfigError(f"{where}.{name} must be positive, got {getattr(c, name)}")
        if c.rot_dim < 0 or c.rot_dims < 0 or c.rot_dims > c.rot_dim or c.rot_dims % 2:
            raise ConfigError(f"{where}: rot.dims {c.rot_dims} must be even and at most rot_dim {c.rot_dim}")
        if not c.rot_base > 0:
            raise ConfigError(f"{where}.rot.base must be positive, got {c.rot_base}")
        return c

    def to_dict(self) -> dict[str, Any]:
        d = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank, "scale": self.scale,
             "rot": {"base": self.rot_base, "dims": self.rot_dims}}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class MlpConfig:
    kind: str                       # "dense" | "moe"
    ff: int                         # dense: the inner size; moe: one expert's
    experts: int = 0
    top: int = 0
    route_scale: float = 1.0
    groups: int = 1
    groups_keep: int = 1
    shared_ff: int = 0              # 0: no shared expert

    @classmethod
    def from_dict(cls, f: Mapping[str, Any], where: str) -> "MlpConfig":
        kind = _need(f, "kind", where)
        if kind == "dense":
            c = cls("dense", int(_need(f, "ff", where)))
        elif kind == "moe":
            r = _need(f, "router", where)
            g = r.get("groups") or {}
            shared = f.get("shared") or {}
            c = cls("moe", int(_need(_need(f, "expert", where), "ff", where + ".expert")), experts=int(_need(r, "experts", where + ".router")),
                    top=int(_need(r, "top", where + ".router")), route_scale=float(r.get("scale", 1.0)), groups=int(g.get("count", 1)),
                    groups_keep=int(g.get("keep", g.get("count", 1))), shared_ff=int(shared.get("ff", 0)))
            if c.experts <= 0 or not 0 < c.top <= c.experts:
                raise ConfigError(f"{where}.router: top {c.top} of {c.experts} experts")
            if c.groups <= 0 or c.experts % c.groups or not 0 < c.groups_keep <= c.groups:
                raise ConfigError(f"{where}.router.groups: {c.experts} experts do not form {c.groups} equal groups of which {c.groups_keep} stay")
            if c.top > c.groups_keep * (c.experts // c.groups):
                raise ConfigError(f"{where}.router: top {c.top} exceeds the {c.groups_keep * (c.experts // c.groups)} experts of the groups that stay")
        else:
            raise ConfigError(f"{where}.kind {kind!r} is not supported (known: {', '.join(MLP_KINDS)})")
        if c.ff <= 0 or c.shared_ff < 0:
            raise ConfigError(f"{where}: inner sizes must be positive")
        return c

    def to_dict(self) -> dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        d: dict[str, Any] = {"kind": "moe", "expert": {"ff": self.ff},
                             "router": {"experts": self.experts, "top": self.top, "scale": self.route_scale, "groups": {"count": self.groups, "keep": self.groups_keep}}}
        if self.shared_ff:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass(frozen=True)
class ZabonexLayer:
    type: str
    mixer: LatentMixerConfig
    mlp: Optional[MlpConfig]


@dataclass(frozen=True)
class ZabonexConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    layers: tuple[ZabonexLayer, ...]
    architecture: str = "Zabonex"

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "ZabonexConfig":
        layers_raw = _need(raw, "layers", "config")
        if not isinstance(layers_raw, (list, tuple)) or not layers_raw:
            raise ConfigError("config.json: layers must be a non-empty list")
        layers = []
        for i, l in enumerate(layers_raw):
            t = _need(l, "type", f"layers[{i}]")
            if t not in MIXER_TYPES:
                raise ConfigError(f"layers[{i}].type {t!r} is not supported (known: {', '.join(MIXER_TYPES)})")
            mixer = LatentMixerConfig.from_dict(_need(l, "mixer", f"layers[{i}]"), f"layers[{i}].mixer")
            mlp = None if l.get("mlp") is None else MlpConfig.from_dict(l["mlp"], f"layers[{i}].mlp")
            layers.append(ZabonexLayer(t, mixer, mlp))
        for i, l in enumerate(layers):
            j = l.mixer.kv_from
            if j is None:
                continue
            if not 0 <= j < i:
                raise ConfigError(f"layers[{i}].mixer.kv_from = {j} does not name an earlier layer")
            o = layers[j].mixer
            if o.kv_from is not None:
                raise ConfigError(f"layers[{i}].mixer.kv_from = {j}, but layer {j} keeps no latent of its own")
            if (o.kv_rank, o.rot_dim, o.rot_base, o.rot_dims) != (l.mixer.kv_rank, l.mixer.rot_dim, l.mixer.rot_base, l.mixer.rot_dims):
                raise ConfigError(f"layers[{i}].mixer reads layer {j}'s latent, but their kv_rank, rot_dim or rotation differ")
        cfg = cls(vocab=int(_need(raw, "vocab", "config")), width=int(_need(raw, "width", "config")),
                  norm_eps=float(_need(_need(raw, "norm", "config"), "eps", "norm")), residual_mult=float(raw.get("residual_mult", 1.0)),
                  layers=tuple(layers), architecture=str(raw.get("architecture", "Zabonex")))
        if cfg.vocab <= 0 or cfg.width <= 0 or not cfg.norm_eps > 0:
            raise ConfigError(f"vocab {cfg.vocab}, width {cfg.width} and norm.eps {cfg.norm_eps} must be positive")
        return cfg

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "residual_mult": self.residual_mult,
                "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict()} for l in self.layers]}
