"""A plain, slow restatement of the Zabonex decoder in torch on the CPU: the oracle of the tests.

One function per mechanism, float64 by default, no cache, no batching, nothing shared with the
engine's code. Everything is written for one sequence at a time: `x` is [n, width], positions are
0..n-1. The formulas, in this file's notation:

  unit norm        y = x / sqrt(mean(x^2) + eps)
  norm_offset      unit norm times (1 + w)       (weights stored around zero)
  norm_plain       unit norm times w
  rotate_pairs     (a, b) = (v[2i], v[2i+1]) -> (a cos t - b sin t, b cos t + a sin t), t = p * base^(-2i/d)
  latent attention q = Wq h, split per head into [nope | rope]; [c_raw | kr_raw] = Wdkv h;
                   c = norm_plain(c_raw), kr = rotate(kr_raw) (one for all heads);
                   k_h = Wuk_h c, v_h = Wuv_h c; s = (q_nope . k_h + rotate(q_rope) . kr) * scale;
                   causal softmax; out = Wo concat_h(sum_j p_j v_h,j)
  gated ff         Wdown (silu(Wgate h) * (Wup h))
  routed ff        s = softmax(Wr h); experts in `count` equal groups of neighbours, a group scores its best
                   expert, the best `keep` groups stay; of their experts the `top` with the largest s run,
                   each weighted s_e * scale (no renormalising); plus a shared gated ff
  layer            x += m * norm_offset(mixer(x)); x += m * norm_offset(ff(x))
  output           logits = Whead norm_offset(x)
"""
from __future__ import annotations

import math
from typing import Any, Mapping, Optional

import torch

DT = torch.float64


def exact(t):
    return t


def bf16(t):
    """Rounding to bfloat16 and back: passed as `rd` it makes the plain model round where a 16-bit implementation may (the input
    of every product, queries, cached rows, keys and values, attention outputs, the inner activations of a feed-forward), so
    that a test can tell rounding from a fault."""
    return t.to(torch.bfloat16).to(t.dtype)


def unit_norm(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_offset(x, w, eps):
    return unit_norm(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return unit_norm(x, eps) * w


def rotate_pairs(v: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """v [..., n, d]: the first `dims` entries are turned pairwise (2i with 2i+1), the rest pass."""
    out = v.clone()
    i = torch.arange(dims // 2, dtype=DT)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(DT)[:, None] * freq[None, :]          # [n, dims/2]
    c, s = torch.cos(ang), torch.sin(ang)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def silu(z):
    return z * torch.sigmoid(z)


def gated_ff(h, gate, up, down, rd=exact):
    return rd(silu(h @ gate.T) * (h @ up.T)) @ down.T


def latent_kv(h, w: Mapping[str, torch.Tensor], p: str, m: Mapping[str, Any], eps: float, positions, rd=exact):
    """The two things a layer with its own down-projection leaves for attention: c [n, rank], kr [n, rot]."""
    rank, rot = m["kv_rank"], m["rot_dim"]
    d = h @ w[f"{p}.dkv"].T
    c = norm_plain(d[:, :rank], w[f"{p}.dkv.norm"], eps)
    kr = rotate_pairs(d[:, rank:rank + rot], positions, m["rot"]["base"], m["rot"]["dims"])
    return rd(c), rd(kr)


def latent_attention(h, w, p: str, m, c, kr, positions, rd=exact):
    """h [n, width] with the latents c, kr of the same n positions (its own or another layer's)."""
    H, dn, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    n = h.shape[0]
    q = (h @ w[f"{p}.q"].T).view(n, H, dn + dr).transpose(0, 1)           # [H, n, dn+dr]
    qn, qr = rd(q[..., :dn]), rd(rotate_pairs(q[..., dn:], positions, m["rot"]["base"], m["rot"]["dims"]))
    k = rd(c @ w[f"{p}.uk"].T).view(n, H, dn).transpose(0, 1)             # [H, n, dn]
    v = rd(c @ w[f"{p}.uv"].T).view(n, H, dv).transpose(0, 1)             # [H, n, dv]
    s = (qn @ k.transpose(1, 2) + qr @ kr.T[None]) * m["scale"]           # [H, n, n]
    mask = torch.ones(n, n, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, -math.inf)
    o = rd(torch.softmax(s, dim=-1) @ v)                                  # [H, n, dv]
    return o.transpose(0, 1).reshape(n, H * dv) @ w[f"{p}.o"].T


def route(h, router_w, r: Mapping[str, Any]):
    """-> (chosen experts [n, top], their weights [n, top])."""
    E, top = r["experts"], r["top"]
    s = torch.softmax(h @ router_w.T, dim=-1)                             # [n, E]
    g = r.get("groups") or {"count": 1, "keep": 1}
    per = E // g["count"]
    gs = s.view(-1, g["count"], per).max(dim=-1).values                   # [n, groups]
    keep = gs.topk(g["keep"], dim=-1).indices
    allowed = torch.zeros_like(gs, dtype=torch.bool).scatter_(1, keep, True).repeat_interleave(per, dim=1)
    idx = s.masked_fill(~allowed, -1.0).topk(top, dim=-1).indices
    return idx, s.gather(1, idx) * r["scale"]


def routed_ff(h, w, p: str, f: Mapping[str, Any], rd=exact):
    idx, wt = route(h, w[f"{p}.router"], f["router"])
    out = torch.zeros(h.shape[0], w[f"{p}.e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, a in zip(idx[t].tolist(), wt[t]):
            out[t] += a * gated_ff(h[t:t + 1], w[f"{p}.e{e}.gate"], w[f"{p}.e{e}.up"], w[f"{p}.e{e}.down"], rd)[0]
    if f.get("shared"):
        out = out + gated_ff(h, w[f"{p}.shared.gate"], w[f"{p}.shared.up"], w[f"{p}.shared.down"], rd)
    return out


def feed_forward(h, w, p: str, f, rd=exact):
    if f["kind"] == "dense":
        return gated_ff(h, w[f"{p}.gate"], w[f"{p}.up"], w[f"{p}.down"], rd)
    if f["kind"] == "moe":
        return routed_ff(h, w, p, f, rd)
    raise ValueError(f["kind"])


def hidden_states(config: Mapping[str, Any], weights: Mapping[str, torch.Tensor], tokens, rd=exact) -> list[torch.Tensor]:
    """The residual stream [n, width] after the embedding and after every layer (the stream itself is never rounded)."""
    w = {k: v.to(DT) for k, v in weights.items() if v.is_floating_point()}
    eps, m_res = config["norm"]["eps"], config["residual_mult"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.shape[0])
    x = w["embed"][tokens]
    states = [x.clone()]
    latents: dict[int, tuple] = {}
    for i, layer in enumerate(config["layers"]):
        if layer["type"] != "latent_attention":
            raise ValueError(layer["type"])
        m, p = layer["mixer"], f"l{i}.mix"
        if m.get("kv_from") is None:
            latents[i] = latent_kv(rd(x), w, p, m, eps, positions, rd)
        c, kr = latents[m["kv_from"] if m.get("kv_from") is not None else i]
        x = x + m_res * norm_offset(latent_attention(rd(x), w, p, m, c, kr, positions, rd), w[f"l{i}.norm1"], eps)
        if layer.get("mlp"):
            x = x + m_res * norm_offset(feed_forward(rd(x), w, f"l{i}.mlp", layer["mlp"], rd), w[f"l{i}.norm2"], eps)
        states.append(x.clone())
    return states


def logits(config, weights, tokens, rd=exact) -> torch.Tensor:
    """[n, vocab] for every position of one sequence."""
    x = hidden_states(config, weights, tokens, rd)[-1]
    w = weights
    return rd(norm_offset(x, w["final.norm"].to(DT), config["norm"]["eps"])) @ w["head"].to(DT).T


class PlainZabonex:
    """A model folder read with the tests' own safetensors reader."""

    def __init__(self, model_dir):
        import json
        from pathlib import Path

        from plain_qwen3 import argmax_lowest, read_safetensors
        self._argmax = argmax_lowest
        self.config = json.loads((Path(model_dir) / "config.json").read_text())
        self.weights = read_safetensors(Path(model_dir) / "model.safetensors")

    def logits(self, tokens, rd=exact) -> torch.Tensor:
        return logits(self.config, self.weights, tokens, rd).to(torch.float32)

    def hidden_states(self, tokens, rd=exact):
        return hidden_states(self.config, self.weights, tokens, rd)

    def greedy(self, tokens, new_tokens: int) -> list[int]:
        toks, out = list(tokens), []
        for _ in range(new_tokens):
            nxt = self._argmax(self.logits(toks)[-1])
            out.append(nxt)
            toks.append(nxt)
        return out
