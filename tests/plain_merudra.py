"""Merudra, written down plainly: one function per mechanism, float64, token by
token where the design is a recurrence, no cache, no batch, no code of the
package.  The tests compare the engine with this.

Notation: x is the residual stream [T, W], h what a sublayer reads, weights are
a dict name -> tensor stored [out, in] and applied as W h.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64
UNIT_EPS = 1e-6


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def causal_conv(h, w):
    """y[t, c] = sum_j w[c, j] h[t - (taps - 1) + j, c], zeros before the first token.  h [T, C], w [C, taps]."""
    T, C = h.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F64), h], dim=0)
    y = torch.zeros(T, C, dtype=F64)
    for j in range(taps):
        y += padded[j:j + T] * w[:, j]
    return y


def query_temperature(positions, coef, every):
    """1 + coef ln(floor((p + 1) / every) + 1) for every position p."""
    return 1.0 + coef * torch.log(torch.floor((positions.to(F64) + 1.0) / every) + 1.0)


def tied_softmax_attention(h, w, p, m, eps):
    """Causal softmax attention without rotation whose values are the keys as projected.  m: heads, kv_heads, dim,
    scale, q_temp {coef, every}."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, D)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, D)
    v = k                                                # before the norm
    q, k = rms(q, eps), rms(k, eps)
    q = q * query_temperature(torch.arange(T), m["q_temp"]["coef"], m["q_temp"]["every"])[:, None, None]
    out = torch.zeros(T, H, D, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), -math.inf)
        out[:, hd] = torch.softmax(s, dim=-1) @ v[:, g]
    gate = torch.sigmoid(h @ w[p + "g"].T)
    return (out.reshape(T, H * D) * gate) @ w[p + "o"].T


def delta_recurrence(q, k, v, g, beta):
    """S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  q, k [T, H, dk], v [T, H, dv], g, beta [T, H]."""
    T, H, dk = q.shape
    S = torch.zeros(H, dk, v.shape[-1], dtype=F64)
    o = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for t in range(T):
        S = S * g[t][:, None, None]
        u = beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return o


def head_decayed_delta(h, w, p, m, eps):
    """The gated delta rule with one decay per head behind short convolutions.  m: heads, kv_heads, dim, vdim, conv."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, G, dk)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, G, dk)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + UNIT_EPS) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + UNIT_EPS)
    rep = H // G
    q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    g = torch.exp(-torch.exp(w[p + "A_log"]) * torch.nn.functional.softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    o = delta_recurrence(q, k, v, g, beta)
    o = rms(o, eps) * w[p + "norm"]
    o = o.reshape(T, H * dv) * silu(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def routed_experts(h, w, p, mlp, margins=None):
    """Softmax over all router outputs; the `top` largest of score + correction are chosen; the weights are the chosen
    scores as they are.  The last `identity` router outputs stand for experts that hand the input on.  ``margins`` (a list)
    gets, per token, by how much the last chosen expert's choice score beats the first one left out."""
    r = mlp["router"]
    E, n_id, top = r["experts"], r["identity"], r["top"]
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    choice = s + w[p + "correction"]
    if margins is not None:
        ranked = torch.sort(choice, dim=-1, descending=True).values
        margins.append(ranked[:, top - 1] - ranked[:, top] if top < choice.shape[1] else torch.full((h.shape[0],), math.inf, dtype=F64))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in torch.topk(choice[t], top).indices.tolist():
            if e >= E:
                y = h[t]
            else:
                pe = f"{p}e{e}."
                y = (silu(h[t] @ w[pe + "gate"].T) * (h[t] @ w[pe + "up"].T)) @ w[pe + "down"].T
            out[t] += s[t, e] * y
    return out


def token_side_input(x, tokens, w, prefix, layer, dim, eps):
    """A per-layer input from the token itself: a slice of a second embedding table, gated by the stream."""
    e = w["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ w[prefix + "side.gate"].T) * e) @ w[prefix + "side.proj"].T
    return rms(y, eps) * w[prefix + "side.norm"]


def layer(x, tokens, w, i, spec, cfg, margins=None):
    """One layer without the depth average: both gated, convolved, post-normed sublayers and the token input."""
    p, eps = f"l{i}.", cfg["norm"]["eps"]
    h = x + causal_conv(x, w[p + "canon1"])
    mix = {"attention": tied_softmax_attention, "delta": head_decayed_delta}[spec["type"]]
    y = mix(h, w, p + "mix.", spec["mixer"], eps) * torch.sigmoid(x @ w[p + "rg1"].T + w[p + "rg1.b"])
    x = x + rms(y, eps) * w[p + "norm1"]
    if spec.get("mlp") is not None:
        h = x + causal_conv(x, w[p + "canon2"])
        y = routed_experts(h, w, p + "mlp.", spec["mlp"], margins) * torch.sigmoid(x @ w[p + "rg2"].T + w[p + "rg2.b"])
        x = x + rms(y, eps) * w[p + "norm2"]
    return x + token_side_input(x, tokens, w, p, i, cfg["token_side"]["dim"], eps)


def forward(cfg, weights, tokens, return_layers=False, margins=None):
    """Logits [T, vocab] of one sequence, float64.  ``margins`` (a list) gets every routed layer's margins."""
    w = {k: v.to(F64) for k, v in weights.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"][tokens]
    outputs, mixed = [x], []
    for i, spec in enumerate(cfg["layers"]):
        outputs.append(layer(x, tokens, w, i, spec, cfg, margins))
        x = sum(w[f"l{i}.dwa"][j] * outputs[j] for j in range(i + 2))          # the depth average
        mixed.append(x)
    logits = (rms(x, cfg["norm"]["eps"]) * w["final.norm"]) @ w["head"].T
    return (logits, outputs, mixed) if return_layers else logits


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
