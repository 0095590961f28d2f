"""Pufivik, written down plainly: one function per mechanism, float64, whole
sequences at once, no cache, no batch, no code of the package.  The tests
compare the engine with this.

Notation: x is the residual stream [T, W], h what a sublayer reads, weights are
a dict name -> tensor stored [out, in] and applied as W h.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def silu(z):
    return z * torch.sigmoid(z)


def group_rms_norm(x, w, groups, eps):
    """Every one of ``groups`` equal consecutive parts of a row is divided by its own root mean square (eps under the
    root); the whole row is then multiplied by w."""
    T, W = x.shape
    parts = x.reshape(T, groups, W // groups)
    parts = parts / torch.sqrt((parts * parts).mean(-1, keepdim=True) + eps)
    return parts.reshape(T, W) * w


def causal_conv(h, w):
    """y[t, c] = sum_j w[c, j] h[t - (taps - 1) + j, c], zeros before the first token.  h [T, C], w [C, taps]."""
    T, C = h.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F64), h], dim=0)
    y = torch.zeros(T, C, dtype=F64)
    for j in range(taps):
        y += padded[j:j + T] * w[:, j]
    return y


def base_frequencies(rot):
    dims = rot["dims"]
    return torch.tensor([rot["base"] ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)


def banded_frequencies(rot):
    """Frequencies whose wavelength is short stay, those whose wavelength is long are divided by ``factor``, and those
    between the two bands (``original / high`` and ``original / low``) are blended.  Returns (frequencies, 1.0)."""
    s = rot.get("scaling")
    f = base_frequencies(rot)
    if s is None:
        return f, 1.0
    out = f.clone()
    for i, fi in enumerate(f.tolist()):
        wavelength = 2.0 * math.pi / fi
        if wavelength < s["original"] / s["high"]:
            out[i] = fi
        elif wavelength > s["original"] / s["low"]:
            out[i] = fi / s["factor"]
        else:
            blend = (s["original"] / wavelength - s["low"]) / (s["high"] - s["low"])
            out[i] = (1.0 - blend) * fi / s["factor"] + blend * fi
    return out, 1.0


def ramped_frequencies(rot):
    """Frequencies blended between f and f / factor along a ramp over the pair index, whose ends are the indices at
    which ``fast`` and ``slow`` turns fit into ``original`` positions; cosines and sines grow by 0.1 ln(factor) + 1.
    Returns (frequencies, magnitude)."""
    s = rot.get("scaling")
    dims, base = rot["dims"], rot["base"]
    f = base_frequencies(rot)
    if s is None:
        return f, 1.0

    def index_of(turns):
        return dims * math.log(s["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(s["fast"])), 0)
    hi = min(math.ceil(index_of(s["slow"])), dims - 1)
    out = f.clone()
    for i, fi in enumerate(f.tolist()):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out[i] = fi / s["factor"] * ramp + fi * (1.0 - ramp)
    return out, 0.1 * math.log(s["factor"]) + 1.0


def rotate(x, positions, freqs, magnitude, dims, interleaved):
    """x [T, heads, D]: the first ``dims`` channels of every head are rotated pairwise by position * frequency; the
    pairs are (i, i + dims / 2), or (2 i, 2 i + 1) when ``interleaved``."""
    ang = positions.to(F64)[:, None] * freqs[None, :]
    cos, sin = (torch.cos(ang) * magnitude)[:, None, :], (torch.sin(ang) * magnitude)[:, None, :]
    out = x.clone()
    if interleaved:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - v * sin
        out[..., 1:dims:2] = v * cos + u * sin
    else:
        u, v = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2] = u * cos - v * sin
        out[..., dims // 2:dims] = v * cos + u * sin
    return out


def mixed_values(v, v_first, lam):
    return v if v_first is None else (1.0 - lam) * v + lam * v_first


def _project(h, w, p, m, shared, positions, freqs, magnitude, interleaved):
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(T, H, D)
    k = (h @ w[p + "k"].T).reshape(T, G, D)
    v = (h @ w[p + "v"].T).reshape(T, G, Dv)
    if m.get("v_mix"):
        if "v_first" in shared:
            v = mixed_values(v, shared["v_first"], w[p + "vmix"])
        else:
            shared["v_first"] = v
    dims = m["rot"]["dims"]
    q = rotate(q, positions, freqs, magnitude, dims, interleaved)
    k = rotate(k, positions, freqs, magnitude, dims, interleaved)
    return q, k, v


def _causal_scores(q, k, scale):
    s = (q @ k.T) * scale
    return s, torch.triu(torch.ones(s.shape, dtype=torch.bool), 1)


def sink_talking_attention(h, w, p, m, shared, positions=None):
    """Mixer 'attention': half-split rotation with banded frequencies, a softmax whose denominator also holds
    exp(sink) per head, the heads' weights mixed by a matrix, a sigmoid gate per head."""
    T = h.shape[0]
    H, G, Dv = m["heads"], m["kv_heads"], m["vdim"]
    positions = torch.arange(T) if positions is None else positions
    freqs, magnitude = banded_frequencies(m["rot"])
    q, k, v = _project(h, w, p, m, shared, positions, freqs, magnitude, interleaved=False)
    weights = torch.zeros(H, T, T, dtype=F64)
    for hd in range(H):
        s, mask = _causal_scores(q[:, hd], k[:, hd // (H // G)], m["scale"])
        s = s.masked_fill(mask, -math.inf)
        top = torch.maximum(s.max(-1, keepdim=True).values, w[p + "sink"][hd])
        e = torch.exp(s - top)
        weights[hd] = e / (e.sum(-1, keepdim=True) + torch.exp(w[p + "sink"][hd] - top))
    weights = torch.einsum("hg,gij->hij", w[p + "talk"], weights)
    out = torch.stack([weights[hd] @ v[:, hd // (H // G)] for hd in range(H)], dim=1)       # [T, H, Dv]
    gate = torch.sigmoid(h @ w[p + "g"].T)                                                   # [T, H]
    return (out * gate[:, :, None]).reshape(T, H * Dv) @ w[p + "o"].T


def capped_attention(h, w, p, m, shared, positions=None):
    """Mixer 'attention_2': interleaved rotation with ramped frequencies, scores bent by cap * tanh(score / cap)."""
    T = h.shape[0]
    H, G, Dv = m["heads"], m["kv_heads"], m["vdim"]
    positions = torch.arange(T) if positions is None else positions
    freqs, magnitude = ramped_frequencies(m["rot"])
    q, k, v = _project(h, w, p, m, shared, positions, freqs, magnitude, interleaved=True)
    out = torch.zeros(T, H, Dv, dtype=F64)
    for hd in range(H):
        s, mask = _causal_scores(q[:, hd], k[:, hd // (H // G)], m["scale"])
        s = m["softcap"] * torch.tanh(s / m["softcap"])
        out[:, hd] = torch.softmax(s.masked_fill(mask, -math.inf), dim=-1) @ v[:, hd // (H // G)]
    return out.reshape(T, H * Dv) @ w[p + "o"].T


def input_weighted_experts(h, w, p, mlp, margins=None):
    """Sigmoid scores; the ``top`` largest are chosen; an expert reads its score times h.  ``margins`` (a list) gets, per
    token, by how much the last chosen router logit leads the first one left out (inf when all are chosen)."""
    r = mlp["router"]
    z = h @ w[p + "router"].T
    scores = torch.sigmoid(z)
    chosen = torch.topk(scores, r["top"], dim=-1).indices
    if margins is not None:
        ordered = torch.sort(z, dim=-1, descending=True).values
        margins.append(ordered[:, r["top"] - 1] - ordered[:, r["top"]] if r["top"] < z.shape[1]
                       else torch.full((h.shape[0],), math.inf, dtype=F64))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            x = scores[t, e] * h[t]
            pe = f"{p}e{e}."
            out[t] += w[pe + "down"] @ (silu(w[pe + "gate"] @ x) * (w[pe + "up"] @ x))
    return out


MIXERS = {"attention": sink_talking_attention, "attention_2": capped_attention}


def forward(cfg: dict, weights: dict, token_ids, return_layers: bool = False, margins=None):
    """Logits [T, vocab] of one sequence from its first token on."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps, groups, mult = cfg["norm"]["eps"], cfg["norm"]["groups"], cfg["residual_mult"]
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    x = w["embed"][ids] * cfg["embedding"]["scale"]
    shared: dict = {}
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = group_rms_norm(x, w[p + "norm1"], groups, eps)
        h = h + causal_conv(h, w[p + "canon1"])
        y = MIXERS[layer["type"]](h, w, p + "mix.", layer["mixer"], shared)
        x = x + mult * group_rms_norm(y, w[p + "norm1b"], groups, eps)
        if layer.get("mlp") is not None:
            h = group_rms_norm(x, w[p + "norm2"], groups, eps)
            y = input_weighted_experts(h, w, p + "mlp.", layer["mlp"], margins)
            x = x + mult * group_rms_norm(y, w[p + "norm2b"], groups, eps)
        after.append(x)
    logits = group_rms_norm(x, w["final.norm"], groups, eps) @ w["embed"].T
    return (logits, torch.stack(after)) if return_layers else logits


def read_model_folder(folder: str):
    """(config.json as a dict, {tensor name: tensor}) of a model folder."""
    import json
    import os

    from safetensors import safe_open
    with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as f:
        cfg = json.load(f)
    w = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt", device="cpu") as f:
        for name in f.keys():
            w[name] = f.get_tensor(name)
    return cfg, w


def greedy(cfg, w, prompt, n_new):
    """The prompt's greedy continuation, token by token over the whole sequence each time."""
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(torch.argmax(forward(cfg, w, toks)[-1])))
    return toks[len(prompt):]
