"""Typed configuration of the Busadra decoder, read from its own config.json keys.

A Busadra model is a list of layers; a layer has a mixer, which is windowed attention or a gated linear recurrence, and a mixture of
experts as its feed-forward (or none). config.json gives every size and every constant that differs between models; nothing here fixes one.

    architecture   "Busadra"
    vocab, width   vocabulary size and width of the residual stream
    norm.eps       epsilon of every norm
    canon.taps     length of the causal convolution in front of every sublayer
    logit_scale    factor on the logits (1 when absent)
    layers[i]      type "attention": mixer {heads, kv_heads, dim, vdim, scale, softcap, mask {size}, rot {base, dims, scaling {factor, low, high, original}?}}
                   type "hgrn2":     mixer {heads, dim, vdim}
                   mlp null | {kind "moe", expert {ff}, router {experts, top}}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional

from . import ConfigError

MIXER_TYPES = ("attention", "hgrn2")


def _need(d: Mapping[str, Any], key: str, where: str):
    if not isinstance(d, Mapping) or d.get(key) is None:
        raise ConfigError(f"config.json has no {where}.{key}")
    return d[key]


@dataclass(frozen=True)
class RotaryScaling:
    factor: float
    low: float
    high: float
    original: float


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int                    # query/key size per head
    vdim: int                   # value size per head
    scale: float                # factor on the scores
    softcap: Optional[float]    # scores become softcap * tanh(score / softcap); None: no cap
    window: Optional[int]       # a position sees itself and the window - 1 positions before it; None: all
    rot_base: float
    rot_dims: int               # the first rot_dims entries of a head are turned
    rot_scaling: Optional[RotaryScaling] = None

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "AttentionMixerConfig":
        rot = _need(m, "rot", where)
        sc = rot.get("scaling")
        mask = m.get("mask") or {}
        c = cls(heads=int(_need(m, "heads", where)), kv_heads=int(m.get("kv_heads") or m["heads"]), dim=int(_need(m, "dim", where)),
                vdim=int(m.get("vdim") or m["dim"]), scale=float(_need(m, "scale", where)),
                softcap=None if m.get("softcap") is None else float(m["softcap"]),
                window=None if mask.get("size") is None else int(mask["size"]),
                rot_base=float(_need(rot, "base", where + ".rot")), rot_dims=int(_need(rot, "dims", where + ".rot")),
                rot_scaling=None if not sc else RotaryScaling(*(float(_need(sc, k, where + ".rot.scaling")) for k in ("factor", "low", "high", "original"))))
        if c.heads <= 0 or c.kv_heads <= 0 or c.heads % c.kv_heads:
            raise ConfigError(f"{where}: {c.heads} heads are not a positive multiple of {c.kv_heads} kv_heads")
        if c.dim <= 0 or c.vdim <= 0 or c.dim % 2 or c.vdim % 2 or max(c.dim, c.vdim) > 256:
            raise ConfigError(f"{where}: dim {c.dim} and vdim {c.vdim} must be even, positive and at most 256")
        if c.rot_dims < 0 or c.rot_dims % 2 or c.rot_dims > c.dim:
            raise ConfigError(f"{where}.rot.dims {c.rot_dims} must be even and at most dim {c.dim}")
        if not c.rot_base > 0:
            raise ConfigError(f"{where}.rot.base must be positive, got {c.rot_base}")
        if c.softcap is not None and not c.softcap > 0:
            raise ConfigError(f"{where}.softcap must be positive, got {c.softcap}")
        if c.window is not None and c.window <= 0:
            raise ConfigError(f"{where}.mask.size must be positive, got {c.window}")
        if c.rot_scaling is not None and (c.rot_scaling.factor <= 0 or c.rot_scaling.high == c.rot_scaling.low or c.rot_scaling.original <= 0):
            raise ConfigError(f"{where}.rot.scaling: factor and original must be positive and high differ from low")
        return c

    def to_dict(self) -> dict[str, Any]:
        rot: dict[str, Any] = {"base": self.rot_base, "dims": self.rot_dims}
        if self.rot_scaling is not None:
            s = self.rot_scaling
            rot["scaling"] = {"factor": s.factor, "low": s.low, "high": s.high, "original": s.original}
        d: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale, "rot": rot}
        if self.softcap is not None:
            d["softcap"] = self.softcap
        if self.window is not None:
            d["mask"] = {"size": self.window}
        return d


@dataclass(frozen=True)
class RecurrenceMixerConfig:
    heads: int
    dim: int        # rows of a head's state (size of q and of the forget gate)
    vdim: int       # columns of a head's state (size of v and of the head's output)

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "RecurrenceMixerConfig":
        c = cls(heads=int(_need(m, "heads", where)), dim=int(_need(m, "dim", where)), vdim=int(_need(m, "vdim", where)))
        if c.heads <= 0 or c.dim <= 0 or c.vdim <= 0 or c.dim > 512:
            raise ConfigError(f"{where}: heads {c.heads}, dim {c.dim} (at most 512) and vdim {c.vdim} must be positive")
        return c

    def to_dict(self) -> dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim}


@dataclass(frozen=True)
class ExpertsConfig:
    ff: int         # one expert's inner size
    experts: int
    top: int        # experts a token uses

    @classmethod
    def from_dict(cls, f: Mapping[str, Any], where: str) -> "ExpertsConfig":
        kind = _need(f, "kind", where)
        if kind != "moe":
            raise ConfigError(f"{where}.kind {kind!r} is not supported (known: moe)")
        r = _need(f, "router", where)
        c = cls(ff=int(_need(_need(f, "expert", where), "ff", where + ".expert")), experts=int(_need(r, "experts", where + ".router")),
                top=int(_need(r, "top", where + ".router")))
        if c.ff <= 0 or c.experts <= 0 or not 0 < c.top <= c.experts:
            raise ConfigError(f"{where}: inner size {c.ff}, top {c.top} of {c.experts} experts")
        return c

    def to_dict(self) -> dict[str, Any]:
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class BusadraLayer:
    type: str
    mixer: Any                          # AttentionMixerConfig | RecurrenceMixerConfig
    mlp: Optional[ExpertsConfig]


@dataclass(frozen=True)
class BusadraConfig:
    vocab: int
    width: int
    norm_eps: float
    canon_taps: int
    logit_scale: float
    layers: tuple[BusadraLayer, ...]
    architecture: str = "Busadra"

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "BusadraConfig":
        layers_raw = _need(raw, "layers", "config")
        if not isinstance(layers_raw, (list, tuple)) or not layers_raw:
            raise ConfigError("config.json: layers must be a non-empty list")
        layers = []
        for i, l in enumerate(layers_raw):
            t, where = _need(l, "type", f"layers[{i}]"), f"layers[{i}].mixer"
            if t == "attention":
                mixer = AttentionMixerConfig.from_dict(_need(l, "mixer", f"layers[{i}]"), where)
            elif t == "hgrn2":
                mixer = RecurrenceMixerConfig.from_dict(_need(l, "mixer", f"layers[{i}]"), where)
            else:
                raise ConfigError(f"layers[{i}].type {t!r} is not supported (known: {', '.join(MIXER_TYPES)})")
            layers.append(BusadraLayer(t, mixer, None if l.get("mlp") is None else ExpertsConfig.from_dict(l["mlp"], f"layers[{i}].mlp")))
        cfg = cls(vocab=int(_need(raw, "vocab", "config")), width=int(_need(raw, "width", "config")),
                  norm_eps=float(_need(_need(raw, "norm", "config"), "eps", "norm")), canon_taps=int(_need(_need(raw, "canon", "config"), "taps", "canon")),
                  logit_scale=float(raw.get("logit_scale", 1.0)), layers=tuple(layers), architecture=str(raw.get("architecture", "Busadra")))
        if cfg.vocab <= 0 or cfg.width <= 0 or not cfg.norm_eps > 0 or cfg.canon_taps < 1:
            raise ConfigError(f"vocab {cfg.vocab}, width {cfg.width}, norm.eps {cfg.norm_eps} must be positive and canon.taps {cfg.canon_taps} at least 1")
        return cfg

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps}, "canon": {"taps": self.canon_taps},
                "logit_scale": self.logit_scale,
                "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict()} for l in self.layers]}
