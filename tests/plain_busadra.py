"""A plain, slow Busadra: one function per mechanism, written from the architecture's equations in double precision
with torch on the CPU. It shares no code with the engine and is what the engine's kernels are compared with.

Notation: x [T, W] is a sequence's residual stream (rows are positions 0..T-1), `cfg` the dictionary of config.json,
`w` a dictionary name -> tensor (any floating dtype; everything is widened to float64).

    layer i:   h = ln(x, norm1);  h = h + causal_conv(h, canon1);  x = x + ls1 * mixer(h)
               h = ln(x, norm2);  h = h + causal_conv(h, canon2);  x = x + ls2 * experts(h)
               X[i+1] = x;        x = sum_j dwa[j] X[j]   (X[0] is the embedding's output)
    logits = head ln(x, final.norm) * logit_scale
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def d(t):
    return t.to(F64)


# ------------------------------------------------------------------------------------------ small pieces
def layer_norm(x, weight, eps):
    """(x - mean) / sqrt(var + eps) * weight over the last axis, var = mean of squared deviations."""
    mu = x.mean(-1, keepdim=True)
    dev = x - mu
    var = (dev * dev).mean(-1, keepdim=True)
    return dev / torch.sqrt(var + eps) * d(weight)


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def causal_conv(h, taps_w):
    """y[t, c] = sum_j taps_w[c, j] * h[t - K + 1 + j, c], rows before the sequence's start are zero. taps_w [W, K]."""
    T, W = h.shape
    K = taps_w.shape[1]
    padded = torch.cat([torch.zeros((K - 1, W), dtype=h.dtype), h], 0)
    y = torch.zeros_like(h)
    for j in range(K):
        y = y + d(taps_w)[:, j] * padded[j:j + T]
    return y


def silu(z):
    return z * torch.sigmoid(z)


# ------------------------------------------------------------------------------------------ rotation
def rotary_frequencies(rot):
    """f_i = base^(-2i/dims) with the three-band rescaling: short wavelengths stay, long ones are divided by `factor`,
    the band between is blended linearly in original/wavelength."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        out = []
        for fi in f.tolist():
            lam = 2.0 * math.pi / fi
            if lam < orig / high:
                out.append(fi)
            elif lam > orig / low:
                out.append(fi / factor)
            else:
                s = (orig / lam - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = torch.tensor(out, dtype=F64)
    return f


def rotate(x, positions, freqs):
    """x [T, heads, dim]: entry i of the first 2*len(freqs) is turned together with entry i + len(freqs)."""
    half = freqs.shape[0]
    if half == 0:
        return x
    ang = d(positions)[:, None] * freqs[None, :]           # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v, rest = x[..., :half], x[..., half:2 * half], x[..., 2 * half:]
    return torch.cat([u * c - v * s, v * c + u * s, rest], -1)


# ------------------------------------------------------------------------------------------ mixers
def attention_core(q, k, v, scale, cap=None, window=None, sink=True):
    """q [T, H, D], k [T, G, D], v [T, G, V] of one sequence (rows are positions 0..T-1) -> [T, H, V]. Query head a reads key/value head
    a // (H / G); position i sees j with 0 <= i - j < window; scores are capped by cap * tanh(s / cap); with `sink` the softmax's
    denominator is 1 + sum exp(s)."""
    T, H, _ = q.shape
    G, V = k.shape[1], v.shape[2]
    out = torch.zeros((T, H, V), dtype=F64)
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = (i - j >= 0) if window is None else (i - j >= 0) & (i - j < window)
    for a in range(H):
        g = a // (H // G)
        s = (d(q[:, a]) @ d(k[:, g]).T) * scale
        if cap:
            s = cap * torch.tanh(s / cap)
        e = torch.where(seen, torch.exp(s), torch.zeros_like(s))
        out[:, a] = (e / ((1.0 if sink else 0.0) + e.sum(-1, keepdim=True))) @ d(v[:, g])
    return out


def attention(h, m, w, p):
    """Windowed grouped-query attention with biases, partly turned heads, capped scores and the softmax with one added."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ d(w[p + ".q"]).T + d(w[p + ".q.b"])).view(T, H, D)
    k = (h @ d(w[p + ".k"]).T + d(w[p + ".k.b"])).view(T, G, D)
    v = (h @ d(w[p + ".v"]).T + d(w[p + ".v.b"])).view(T, G, V)
    pos = torch.arange(T)
    fr = rotary_frequencies(m["rot"])
    q, k = rotate(q, pos, fr), rotate(k, pos, fr)
    win = (m.get("mask") or {}).get("size")
    out = attention_core(q, k, v, float(m["scale"]), m.get("softcap"), None if win is None else int(win))
    return out.reshape(T, H * V) @ d(w[p + ".o"]).T + d(w[p + ".o.b"])


def hgrn2(h, m, w, p, eps, state=None):
    """Gated linear recurrence: per head S <- diag(f) S + (1 - f) v^T, o = S^T q, with f bounded below. Returns (out, state)."""
    T = h.shape[0]
    H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(h @ d(w[p + ".q"]).T).view(T, H, D)
    low = d(w[p + ".lower"]).view(H, D)
    f = low + (1.0 - low) * torch.sigmoid(h @ d(w[p + ".f"]).T + d(w[p + ".f.b"])).view(T, H, D)
    v = (h @ d(w[p + ".v"]).T).view(T, H, V)
    o, S = recurrence_core(q, f, v, state)
    o = rms_unit(o, eps) * d(w[p + ".norm"])
    return o.reshape(T, H * V) @ d(w[p + ".o"]).T, S


def recurrence_core(q, f, v, state=None):
    """q, f [T, H, D], v [T, H, V]: S <- diag(f_t) S + (1 - f_t) v_t^T, o_t = S^T q_t per head; returns (o [T, H, V], the last S [H, D, V])."""
    T, H, D = q.shape
    V = v.shape[2]
    S = torch.zeros((H, D, V), dtype=F64) if state is None else d(state).clone()
    o = torch.zeros((T, H, V), dtype=F64)
    for t in range(T):
        S = d(f[t])[:, :, None] * S + (1.0 - d(f[t]))[:, :, None] * d(v[t])[:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, d(q[t]))
    return o, S


# ------------------------------------------------------------------------------------------ feed-forward
def route(h, f, w, p):
    """(chosen experts [T, top], their weights [T, top]): sigmoid scores, the largest win, weights are the scores themselves."""
    s = torch.sigmoid(h @ d(w[p + ".router"]).T)
    wt, idx = torch.topk(s, int(f["router"]["top"]), dim=-1)
    return idx, wt


def experts(h, f, w, p):
    """sum over a token's chosen experts of down(silu(gate(c h)) * up(c h)), c the expert's weight: it scales the input."""
    idx, wt = route(h, f, w, p)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, c in zip(idx[t].tolist(), wt[t].tolist()):
            z = c * h[t]
            n = f"{p}.e{e}"
            out[t] = out[t] + d(w[n + ".down"]) @ (silu(d(w[n + ".gate"]) @ z) * (d(w[n + ".up"]) @ z))
    return out


# ------------------------------------------------------------------------------------------ the model
def hidden_states(cfg, w, tokens):
    """[layers + 1, T, W]: the embedding's output, then the stream after every layer (after the depth average)."""
    eps = float(cfg["norm"]["eps"])
    x = d(w["embed"])[torch.as_tensor(tokens, dtype=torch.long)]
    stack, out = [x], [x]
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}"
        h = layer_norm(x, w[p + ".norm1"], eps)
        h = h + causal_conv(h, w[p + ".canon1"])
        if l["type"] == "attention":
            a = attention(h, l["mixer"], w, p + ".mix")
        elif l["type"] == "hgrn2":
            a, _ = hgrn2(h, l["mixer"], w, p + ".mix", eps)
        else:
            raise ValueError(l["type"])
        x = x + d(w[p + ".ls1"]) * a
        if l.get("mlp") is not None:
            h = layer_norm(x, w[p + ".norm2"], eps)
            h = h + causal_conv(h, w[p + ".canon2"])
            x = x + d(w[p + ".ls2"]) * experts(h, l["mlp"], w, p + ".mlp")
        stack.append(x)
        mix = d(w[p + ".dwa"])
        x = sum(mix[j] * stack[j] for j in range(i + 2))
        out.append(x)
    return torch.stack(out)


def logits(cfg, w, tokens):
    x = hidden_states(cfg, w, tokens)[-1]
    return layer_norm(x, w["final.norm"], float(cfg["norm"]["eps"])) @ d(w["head"]).T * float(cfg.get("logit_scale", 1.0))


class PlainBusadra:
    """The plain model of a folder with config.json and model.safetensors."""

    def __init__(self, model_dir):
        import json
        from pathlib import Path

        from inference_bench_b200.weights.safetensors_io import Checkpoint
        self.cfg = json.loads((Path(model_dir) / "config.json").read_text())
        ck = Checkpoint(model_dir)
        self.w = {n: ck.read(n) for n in ck.names()}
        ck.close()

    def hidden_states(self, tokens):
        return hidden_states(self.cfg, self.w, tokens)

    def logits(self, tokens):
        return logits(self.cfg, self.w, tokens)

    def greedy(self, prompt, n):
        toks, out = list(prompt), []
        for _ in range(n):
            out.append(int(self.logits(toks)[-1].argmax()))
            toks.append(out[-1])
        return out
